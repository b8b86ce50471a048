"""Per-expert restatement of the reference's torch oracle (test infrastructure only).

Every function names the reference lines it follows (paths relative to the
ROCm/aiter tree).  The reference dequantises all experts to fp32 at once
(``aiter/fused_moe.py:3581,3589-3594,3724,3737-3743``), ~60 GB for a
DeepSeek-V3 ``w1``; here the same element-wise arithmetic and the same
``sub_tokens @ w_e.T`` matmuls are issued one expert at a time, which is
bit-identical on CPU (checked by ``tests/golden/make_golden.py``).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0  # torch.finfo(float8_e4m3fn).max


# --------------------------------------------------------------------------- quantisers
def _pertoken_quant(x: torch.Tensor, quant_dtype=FP8):
    """aiter/ops/quant.py:64-94 (pertoken_quant, scale=None, x_scale=None).

    amax over the last dim -> scale = amax / dtypeMax (true division), zero
    scales become 1, codes = (x / scale) cast to the quant dtype (RNE).
    """
    x = x.to(torch.float32)
    amax, _ = torch.max(torch.abs(x), dim=-1, keepdim=True)
    scale = amax / FP8_MAX
    scale[scale == 0] = 1
    y = (x / scale).to(dtype=quant_dtype)
    return y, scale.to(torch.float32)


def quant_1x128(x: torch.Tensor):
    """1x128 activation quant as the 2-stage test does it:
    op_tests/test_moe_2stage.py:237-242 (a1) and :419-423 (a2).
    ``x`` [R, C] -> codes [R, C] e4m3, scales [R, C/128] fp32."""
    R, C = x.shape
    q, s = _pertoken_quant(x.reshape(R, -1, 128))
    return q.view(R, C), s.squeeze(-1)


def quant_weight_128x128(w: torch.Tensor):
    """op_tests/test_moe_2stage.py:184-208 (weight_per_128x128_quant).
    ``w`` [E, N, K] -> codes [E, N, K] e4m3, scales [E, N/128, K/128] fp32."""
    E, d1, d2 = w.shape
    blocks = w.view(E, d1 // 128, 128, d2 // 128, 128).permute(0, 1, 3, 2, 4).contiguous()
    blocks = blocks.view(E, -1, 128 * 128)
    q, s = _pertoken_quant(blocks)
    q = q.view(E, d1 // 128, d2 // 128, 128, 128).permute(0, 1, 3, 2, 4).contiguous()
    return q.view(E, d1, d2), s.view(E, d1 // 128, d2 // 128)


def quant_per_token(x: torch.Tensor):
    """get_torch_quant(per_Token): pertoken_quant over the last dim
    (aiter/ops/quant.py:349-364; used by op_tests/test_moe_2stage.py:213-214,264)."""
    return _pertoken_quant(x)


# --------------------------------------------------------------------------- sorting
def quant_per_tensor(x: torch.Tensor):
    """per_tensor_quant (aiter/ops/quant.py:318-328): one scale = max|x| / 448 for the whole tensor, codes =
    (x / scale).to(e4m3); no guard for an all-zero tensor. Returns (codes, scale [1])."""
    x32 = x.to(torch.float32)
    scale = torch.abs(x32).max() / 448.0
    return (x32 / scale).to(FP8), scale.view(1).to(torch.float32)


def moe_sorting_ref(topk_ids, topk_weights, num_experts, block_size,
                    expert_mask=None, num_local_tokens=None):
    """op_tests/test_moe_sorting.py:45-99 (run_torch_moe_sorting).

    Stable bucket sort of (token, slot) by expert, each expert padded to a
    multiple of ``block_size``; ids pack ``slot << 24 | token``; pad entries are
    ``topk << 24 | M`` with M the static row count; experts without routes get
    no block; masked experts are dropped and the rest renumbered.
    Slots that the reference leaves unwritten (weights of pads, ids past the
    padded total) are returned as 0.0 / pad-id / -1."""
    m, topk = topk_ids.shape
    max_padded = topk_ids.numel() + num_experts * block_size - topk
    max_blocks = (max_padded + block_size - 1) // block_size
    init_val = topk << 24 | m
    sorted_ids = torch.full((max_padded,), init_val, dtype=torch.int32)
    sorted_weights = torch.zeros((max_padded,), dtype=torch.float32)
    sorted_expert_ids = torch.full((max_blocks,), -1, dtype=torch.int32)
    num_valid = torch.empty((2,), dtype=torch.int32)
    if num_local_tokens is not None:
        topk_ids = topk_ids[: int(num_local_tokens.item())]
    begin = 0
    blk_begin = 0
    skipped = 0
    for e in range(num_experts):
        if expert_mask is not None and int(expert_mask[e]) == 0:
            skipped += 1
            continue
        token_id, slot_id = torch.where(topk_ids == e)
        n = token_id.numel()
        nblk = (n + block_size - 1) // block_size
        sorted_ids[begin:begin + n] = (slot_id << 24 | token_id).to(torch.int32)
        sorted_weights[begin:begin + n] = topk_weights[token_id, slot_id]
        begin += nblk * block_size
        sorted_expert_ids[blk_begin:blk_begin + nblk] = e - skipped
        blk_begin += nblk
    num_valid[0] = begin
    num_valid[1] = topk_ids.shape[0]
    return sorted_ids, sorted_weights, sorted_expert_ids, num_valid


def local_expert_ids(topk_ids, expert_mask):
    """aiter/fused_moe.py:3467-3470: local id = cumsum(mask) - 1, non-local -> -1."""
    if expert_mask is None:
        return topk_ids
    mask = expert_mask.to(torch.int64)
    local = torch.cumsum(mask, 0) - 1
    local = torch.where(mask > 0, local, torch.full_like(local, -1))
    return local[topk_ids.long()].to(topk_ids.dtype)


# --------------------------------------------------------------------------- GEMM stages
def _dequant_expert(w_q_e, w_s_e, per_token=False):
    """aiter/fused_moe.py:3589-3594: w.view(N/128,128,K/128,128) * scale.view(N/128,1,K/128,1);
    per_Token (:3583-3585): w * scale.view(N, 1)."""
    N, K = w_q_e.shape
    if per_token:   # [N] scales per output channel, or one scale for the expert (per_Tensor)
        return w_q_e.to(torch.float32) * w_s_e.reshape(-1, 1)
    w = w_q_e.to(torch.float32).view(N // 128, 128, K // 128, 128)
    w = w * w_s_e.reshape(N // 128, 1, K // 128, 1)
    return w.view(N, K)


def moe_stage1_ref(a1_q, a1_scale, w1_q, w1_scale, topk_weight, topk_ids, inter_dim,
                   dtype=torch.bfloat16, doweight=False, per_token=False, activation="silu"):
    """aiter/fused_moe.py:3532-3681, per_1x128/per_128x128 branch, g1u1, SiLU.

    a1_q [M,H] e4m3 + a1_scale [M,H/128]; w1_q [E,2I,H] e4m3 + w1_scale
    [E,2I/128,H/128]; topk_ids hold *local* expert ids (-1 = not on this rank).
    Returns [M, topk, I] in ``dtype`` (rows of non-local routes are 0)."""
    M, H = a1_q.shape
    topk = topk_ids.shape[1]
    E, N, _ = w1_q.shape
    hidden = a1_q.to(torch.float32)
    if per_token:   # aiter/fused_moe.py:3583-3585: hidden_states * a1_scale with a1_scale [M, 1]
        hidden = hidden * a1_scale.reshape(-1, 1)   # [M,1], or [1] for per_Tensor
    else:
        s = a1_scale.view(M, -1, 1).repeat(1, 1, H // a1_scale.view(M, -1).shape[1]).view(M, -1)
        hidden = hidden * s
    out = torch.zeros((M, topk, N), dtype=torch.float32)
    for e in range(E):
        mask = topk_ids == e
        if mask.sum():
            tok, _slot = torch.where(mask)
            sub = hidden[tok]
            w_e = _dequant_expert(w1_q[e], w1_scale[e], per_token)
            act_in = sub @ w_e.transpose(0, 1)
            if doweight:
                act_in = act_in * topk_weight[mask].view(-1, 1)
            out[mask] = act_in
    act = F.gelu if activation == "gelu" else F.silu   # aiter.get_torch_act (aiter/fused_moe.py:3665)
    if N == 2 * inter_dim:
        gate, up = out.split([inter_dim, inter_dim], dim=-1)
        out = act(gate) * up
    else:
        out = act(out)
    return out.to(dtype)


def moe_stage2_ref(a2_q, a2_scale, w2_q, w2_scale, topk_weight, topk_ids,
                   dtype=torch.bfloat16, doweight=True, per_token=False):
    """aiter/fused_moe.py:3684-3811, per_1x128/per_128x128 branch.

    a2_q [M,topk,I] e4m3 + a2_scale [M,topk,I/128]; w2_q [E,H,I] + w2_scale
    [E,H/128,I/128].  fp32 per-route results, times the route weight, summed
    over top-k in fp32, one final cast."""
    M, topk = topk_ids.shape
    E, H, I = w2_q.shape
    hidden = a2_q.to(torch.float32).view(M, topk, I)
    if per_token:   # aiter/fused_moe.py:3729-3731: a2_scale [M, topk, 1]
        hidden = hidden * (a2_scale.reshape(1, 1, 1) if a2_scale.numel() == 1 else a2_scale.view(M, topk, 1))
    else:
        s = a2_scale.view(M, topk, -1, 1).repeat(1, 1, 1, 128).view(M, topk, -1)
        hidden = hidden * s
    out = torch.zeros((M, topk, H), dtype=torch.float32)
    for e in range(E):
        mask = topk_ids == e
        if mask.sum():
            sub = hidden[mask]
            w_e = _dequant_expert(w2_q[e], w2_scale[e], per_token)
            out[mask] = sub @ w_e.transpose(0, 1)
    if doweight:
        out.mul_(topk_weight.view(M, -1, 1))
    return out.sum(1).to(dtype)


def fused_moe_ref(x, w1_q, w1_scale, w2_q, w2_scale, topk_weight, topk_ids,
                  expert_mask=None, dtype=torch.bfloat16, return_stages=False,
                  a1_q=None, a1_scale=None, per_token=False, activation="silu",
                  doweight_stage1=False, per_tensor=False):
    """The pipeline of op_tests/test_moe_2stage.py (per_128x128 branch):
    a1 quant :237-242 -> torch_moe_stage1 :397-416 -> a2 quant :419-423 ->
    torch_moe_stage2 :448-460.  ``expert_mask`` follows torch_moe
    (aiter/fused_moe.py:3467-3470)."""
    M, H = x.shape
    I = w2_q.shape[2]
    ids = local_expert_ids(topk_ids, expert_mask)
    quant = quant_per_token if per_token else quant_1x128   # per_Token: op_tests/test_moe_2stage.py:264,446
    if per_tensor:   # per_Tensor shares per_Token's dequantisation (aiter/fused_moe.py:3583-3585, 3729-3731)
        quant, per_token = quant_per_tensor, True
    if a1_q is None:
        a1_q, a1_scale = quant(x)
    out1 = moe_stage1_ref(a1_q, a1_scale, w1_q, w1_scale, topk_weight, ids, I, dtype=dtype, per_token=per_token,
                          activation=activation, doweight=doweight_stage1)
    a2_q, a2_scale = quant(out1.view(-1, I))
    topk = topk_ids.shape[1]
    out = moe_stage2_ref(a2_q.view(M, topk, I), a2_scale if per_tensor else a2_scale.view(M, topk, -1), w2_q, w2_scale,
                         topk_weight, ids, dtype=dtype, per_token=per_token, doweight=not doweight_stage1)
    if return_stages:
        return out, dict(a1_q=a1_q, a1_scale=a1_scale, out1=out1, a2_q=a2_q.view(M, topk, I),
                         a2_scale=a2_scale if per_tensor else a2_scale.view(M, topk, -1))
    return out


# --------------------------------------------------------------------------- routing
def softmax_topk_ref(logits, topk, renormalize=True):
    """aiter/fused_moe.py:4058-4129 (fused_topk): fp32 softmax, top-k, renormalise."""
    scores = torch.softmax(logits.to(torch.float32), dim=-1)
    w, ids = torch.topk(scores, k=topk, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(torch.float32), ids.to(torch.int32)


def biased_grouped_topk_ref(gating, bias, topk, renormalize, num_expert_group, topk_group,
                            routed_scaling_factor=1.0):
    """aiter/ops/topk.py:217-259 (biased_grouped_topk_torch) followed by the
    routed_scaling_factor multiply of the native op (aiter/ops/topk.py:90-99)."""
    scores = gating.to(torch.float32).sigmoid()
    n = scores.shape[0]
    choice = scores.view(n, -1) + bias.unsqueeze(0)
    group_scores = choice.view(n, num_expert_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
    group_idx = torch.topk(group_scores, k=topk_group, dim=-1, sorted=False)[1]
    group_mask = torch.zeros_like(group_scores)
    group_mask.scatter_(1, group_idx, 1)
    score_mask = (group_mask.unsqueeze(-1)
                  .expand(n, num_expert_group, scores.shape[-1] // num_expert_group)
                  .reshape(n, -1))
    tmp = choice.masked_fill(~score_mask.bool(), 0.0)
    _, ids = torch.topk(tmp, k=topk, dim=-1, sorted=False)
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    w = w * routed_scaling_factor
    return w.to(torch.float32), ids.to(torch.int32)


# --------------------------------------------------------------------------- error metrics
def error_stats(out: torch.Tensor, ref: torch.Tensor, atol=1e-2, rtol=1e-2):
    """Parity statistics for a bf16 output against the oracle.

    max_abs_over_rms: max |out-ref| / RMS(ref)   (bar: <= 0.02)
    frac_within:      share of elements with |out-ref| <= atol + rtol*|ref|  (bar: >= 0.995)
    n_diff / n_one_ulp: elements that differ at all / by exactly one bf16 ulp.
    max_abs_excl_one_ulp_over_rms: the first figure over the elements that are NOT exact one-ulp
    neighbours of the reference. One bf16 ulp of an element above ~2.6 RMS is already more than
    2 % of RMS, so at millions of outputs a single flipped final rounding on a large element
    decides the strict figure; this one shows what is left beside such flips.
    n_two_steps: elements two representable bf16 values away from the reference; max_bf16_steps: the largest such
    distance over same-sign pairs (large for values next to zero, where it means nothing)."""
    o = out.detach().to("cpu", torch.float32)
    r = ref.detach().to("cpu", torch.float32)
    d = (o - r).abs()
    rms = float(r.pow(2).mean().sqrt())
    within = float((d <= atol + rtol * r.abs()).float().mean())
    n_diff = int((d > 0).sum())
    n_one_ulp = 0
    n_two_steps = 0
    max_steps = None
    max_excl = float(d.max())
    if out.dtype == torch.bfloat16 and ref.dtype == torch.bfloat16:
        ob = out.detach().cpu().view(torch.int16).to(torch.int32)
        rb = ref.detach().cpu().view(torch.int16).to(torch.int32)
        steps = (ob - rb).abs()             # distance in representable bf16 values (same sign)
        one = steps == 1                    # neighbouring bf16 values: one final rounding flipped
        n_one_ulp = int(one.sum())
        n_two_steps = int((steps == 2).sum())
        same_sign = (ob ^ rb) >= 0
        max_steps = int(steps[same_sign].max()) if bool(same_sign.any()) else 0
        max_excl = float(d.masked_fill(one, 0.0).max())
    return dict(max_abs=float(d.max()), rms=rms,
                max_abs_over_rms=float(d.max()) / max(rms, 1e-30),
                max_abs_excl_one_ulp_over_rms=max_excl / max(rms, 1e-30),
                frac_within=within, n_diff=n_diff, n_one_ulp=n_one_ulp, n_two_steps=n_two_steps,
                max_bf16_steps=max_steps, numel=o.numel(), has_nan=bool(torch.isnan(o).any()))
