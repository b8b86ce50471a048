"""Host side of the FP8 block-scaled fused-MoE path, behind the reference's own signatures.

``fused_moe`` and ``moe_sorting`` keep the names, argument order and defaults of
aiter/fused_moe.py:458-494 and :341-355, so a caller written for the reference runs unchanged.
Everything that computes is a hand-written sm_100a kernel reached through the C-ABI of
libaiter_b200.so (``_lib.call``); torch is used for device memory and streams only.  There is no
tuned-config dispatch and no fallback: options outside the FP8 1x128 / 128x128 path raise
``NotImplementedError`` naming the argument.
"""

from __future__ import annotations

import os

import torch

from . import _lib
from . import dtypes
from .enums import ActivationType, QuantType

BLOCK_SIZE_M = 32          # default padding unit of moe_sorting (aiter/fused_moe.py:63)
GEMM_BLOCK_M = 128         # row tile of the tcgen05 GEMM kernels == sort unit used by fused_moe

# aiter/fused_moe.py:1310
quant_remap = {QuantType.per_128x128: QuantType.per_1x128}

_status_words: dict[int, torch.Tensor] = {}
_CHECK_STATUS_EVERY_CALL = os.environ.get("AITER_B200_CHECK_STATUS", "0") not in ("", "0")


def _status(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the GEMM kernels set if a bounded device-side wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[idx]


def check_device_status(device=None) -> None:
    """Synchronises and raises if a kernel reported a timed-out wait since the last check."""
    for idx, word in list(_status_words.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        if int(word.item()) != 0:
            word.zero_()
            raise RuntimeError("aiter_b200: a GEMM kernel gave up on a device-side wait "
                               f"(cuda:{idx}); its output is incomplete")


# ------------------------------------------------------------------------------------- sorting
def moe_sorting_get_workspace_size(tokens: int, num_experts: int, topk: int, dispatch_policy: int = 0) -> int:
    """aiter/ops/moe_sorting_opus.py:12-18."""
    return int(_lib.lib().b200_moe_sorting_get_workspace_size(int(tokens), int(num_experts), int(topk),
                                                              int(dispatch_policy)))


def moe_sorting(
    topk_ids,
    topk_weights,
    num_experts,
    model_dim,
    moebuf_dtype,
    block_size=BLOCK_SIZE_M,
    expert_mask=None,
    num_local_tokens=None,
    dispatch_policy=0,
    return_local_topk_ids=False,
    accumulate=True,
    flat=False,
    output_aux=False,
):
    """aiter/fused_moe.py:341-406 / _moe_sorting_impl :175-288.

    Returns (sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids, moe_buf)
    (+ local_topk_ids when asked).  moe_buf is [M, model_dim] and zero-filled when
    ``accumulate`` or ``expert_mask`` is given, else a (0, 0) placeholder."""
    if flat:
        raise NotImplementedError("moe_sorting: flat=True (unsorted pass-through) is not supported")
    if output_aux:
        raise NotImplementedError("moe_sorting: output_aux=True is not supported")
    return _moe_sorting_impl(topk_ids, topk_weights, num_experts, model_dim, moebuf_dtype, block_size,
                             expert_mask, num_local_tokens, dispatch_policy, return_local_topk_ids,
                             want_moe_buf=(expert_mask is not None) or accumulate)


def _moe_sorting_impl(topk_ids, topk_weights, num_experts, model_dim, moebuf_dtype, block_size, expert_mask,
                      num_local_tokens, dispatch_policy, return_local_topk_ids, want_moe_buf):
    """aiter/fused_moe.py:175-288: allocates the outputs and calls the native sort."""
    if not topk_ids.is_cuda:
        raise RuntimeError("moe_sorting: topk_ids must be a CUDA tensor (there is no CPU path)")
    device = topk_ids.device
    M, topk = topk_ids.shape
    block_size = int(block_size)
    max_num_tokens_padded = int(topk_ids.numel() + num_experts * block_size - topk)
    max_num_m_blocks = int((max_num_tokens_padded + block_size - 1) // block_size)
    sorted_ids = torch.empty(max_num_tokens_padded, dtype=dtypes.i32, device=device)
    sorted_weights = torch.empty(max_num_tokens_padded, dtype=dtypes.fp32, device=device)
    sorted_expert_ids = torch.empty(max_num_m_blocks, dtype=dtypes.i32, device=device)
    num_valid_ids = torch.empty(2, dtype=dtypes.i32, device=device)
    if want_moe_buf:
        moe_buf = torch.empty((M, model_dim), dtype=moebuf_dtype, device=device)
    else:
        moe_buf = torch.empty((0, 0), dtype=moebuf_dtype, device=device)
    local_topk_ids = torch.empty_like(topk_ids) if return_local_topk_ids else None
    ws_size = moe_sorting_get_workspace_size(M, num_experts, topk)
    workspace = torch.empty(ws_size, dtype=torch.uint8, device=device) if ws_size > 0 else None
    _lib.call(
        "b200_moe_sorting_fwd",
        topk_ids.contiguous(), topk_weights.contiguous(), sorted_ids, sorted_weights, sorted_expert_ids,
        num_valid_ids, moe_buf if moe_buf.numel() > 0 else None, int(num_experts), block_size,
        expert_mask, num_local_tokens, workspace, int(dispatch_policy), local_topk_ids, None, None,
        device=device,
    )
    ret = (sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids, moe_buf)
    if return_local_topk_ids:
        return (*ret, local_topk_ids)
    return ret


# ------------------------------------------------------------------------------------- quant
_ACT_DTYPES = (dtypes.bf16, dtypes.fp16)


def _check_quant_args(fn, x, scale, quant_dtype):
    if scale is not None:
        # aiter/ops/quant.py:419-420, 454-455: the reference raises the same way
        raise ValueError("unsupported: static per token quant")
    if quant_dtype != dtypes.fp8:
        raise NotImplementedError(f"{fn}: quant_dtype={quant_dtype} is not supported, only dtypes.fp8 (e4m3fn); "
                                  "pass quant_dtype=dtypes.fp8 (the reference's default is dtypes.i8)")
    if x.dtype not in _ACT_DTYPES:
        raise NotImplementedError(f"{fn}: input must be bf16 or fp16, got {x.dtype}")
    if not x.is_cuda:
        raise RuntimeError(f"{fn}: input must be a CUDA tensor (there is no CPU path)")


def per_group_quant_hip(x, scale=None, quant_dtype=dtypes.i8, group_size=128, transpose_scale=False,
                        num_rows=None, num_rows_factor=1, scale_type=dtypes.fp32):
    """Per-row, per-128-column dynamic FP8 quantisation; parameter list of aiter/ops/quant.py:439-448.

    x [..., C] bf16|fp16 -> (codes [..., C] e4m3, scales [..., C/128] fp32). ``num_rows``: device int32 [1],
    only the first num_rows*num_rows_factor rows are written. ``transpose_scale``: the scale buffer keeps its
    shape but holds the [C/128, rows] transpose (the layout the reference's 1-stage kernels read,
    aiter/fused_moe.py:1138-1147). Only quant_dtype=dtypes.fp8, group_size=128 and fp32 scales exist here."""
    _check_quant_args("per_group_quant_hip", x, scale, quant_dtype)
    if group_size != 128:
        raise NotImplementedError(f"per_group_quant_hip: group_size={group_size} is not supported, only 128")
    if scale_type != dtypes.fp32:
        raise NotImplementedError(f"per_group_quant_hip: scale_type={scale_type} is not supported, only fp32")
    x = x.contiguous()
    cols = x.shape[-1]
    y = torch.empty(x.shape, dtype=dtypes.fp8, device=x.device)
    y_scale = torch.empty((*x.shape[:-1], cols // 128), dtype=dtypes.fp32, device=x.device)
    _lib.call("b200_moe_quant_1x128", y, x, y_scale, num_rows, int(num_rows_factor), int(bool(transpose_scale)),
              device=x.device)
    return y, y_scale


def per_token_quant_hip(x, scale=None, quant_dtype=dtypes.i8, num_rows=None, num_rows_factor=1):
    """Per-row dynamic FP8 quantisation; parameter list of aiter/ops/quant.py:406-413.
    x [..., C] bf16|fp16 -> (codes [..., C] e4m3, scales [..., 1] fp32). ``num_rows``: device int32 [1]; rows at or
    past num_rows*num_rows_factor are left untouched. Only quant_dtype=dtypes.fp8 exists here."""
    _check_quant_args("per_token_quant_hip", x, scale, quant_dtype)
    x = x.contiguous()
    cols = x.shape[-1]
    x2 = x.view(-1, cols)
    y = torch.empty(x2.shape, dtype=dtypes.fp8, device=x.device)
    y_scale = torch.empty((x2.shape[0],), dtype=dtypes.fp32, device=x.device)
    _lib.call("b200_moe_quant_per_token", y, x2, y_scale, num_rows, int(num_rows_factor), device=x.device)
    return y.view(x.shape), y_scale.view(*x.shape[:-1], 1)


def _per_tensor_quant(x, row_limit=None, want_row_scales=False):
    """Dynamic per-tensor FP8 quantisation with the two extras the layer needs: ``row_limit`` (device int32 [1],
    rows at or past it take no part) and the scale repeated once per row (what the GEMM kernels read)."""
    x = x.contiguous()
    x2 = x.view(-1, x.shape[-1])
    y = torch.empty(x2.shape, dtype=dtypes.fp8, device=x.device)
    y_scale = torch.empty((1,), dtype=dtypes.fp32, device=x.device)
    amax = torch.empty((1,), dtype=dtypes.fp32, device=x.device)
    rows = torch.empty((x2.shape[0],), dtype=dtypes.fp32, device=x.device) if want_row_scales else None
    _lib.call("b200_moe_quant_per_tensor", y, x2, y_scale, amax, rows, row_limit, device=x.device)
    return y.view(x.shape), y_scale, rows


def per_tensor_quant_hip(x, scale=None, quant_dtype=dtypes.i8, num_rows=None, num_rows_factor=1):
    """Per-tensor dynamic FP8 quantisation; parameter list of aiter/ops/quant.py:628-634.
    x [..., C] bf16|fp16 -> (codes e4m3, scale [1] fp32). Like the reference, ``num_rows`` is not supported."""
    assert num_rows is None, "num_rows is not supported for per_tensor_quant_hip"   # aiter/ops/quant.py:635
    if scale is not None:
        raise NotImplementedError("per_tensor_quant_hip: static quantisation (scale=...) is not supported")
    _check_quant_args("per_tensor_quant_hip", x, None, quant_dtype)
    y, y_scale, _ = _per_tensor_quant(x)
    return y, y_scale.view(1)


def get_hip_quant(qType):
    """aiter/ops/quant.py:367-387, restricted to the FP8 paths built here. Like the reference's table, the
    per_1x128 entry is ``per_group_quant_hip`` with group_size bound to 128, so callers can pass ``transpose_scale``,
    ``num_rows`` and ``num_rows_factor`` (aiter/fused_moe.py:1138-1147)."""
    import functools
    qType = quant_remap.get(QuantType(qType), QuantType(qType))
    if qType == QuantType.per_Token:
        return per_token_quant_hip
    if qType == QuantType.per_Tensor:
        return per_tensor_quant_hip
    if qType != QuantType.per_1x128:
        raise NotImplementedError(f"get_hip_quant: only per_1x128 / per_128x128 / per_Token / per_Tensor are supported, got {qType!r}")
    return functools.partial(per_group_quant_hip, group_size=128)


# ------------------------------------------------------------------------------------- fused_moe
def _check_unsupported(**kw):
    for name, (value, neutral) in kw.items():
        bad = (value is not None) if neutral is None else (value != neutral)
        if bad:
            raise NotImplementedError(f"fused_moe: {name}={value!r} is not supported by the B200 "
                                      "FP8 block-scale path")


def _fold_shared_expert(w1, w2, w1_scale, w2_scale, shared, shared_expert_id, quant_type, expert_mask):
    """Separate shared-expert weights (the ``shared_*`` arguments of aiter/fused_moe.py:488-493).

    The calling contract is the reference's (aiter/fhmoe.py:36-47, 74-98): all four tensors together, the routed
    weights carry a dummy final row, ``shared_expert_id == E - 1``, ``shared_w1 [1, 2I, H]`` / ``shared_w2 [1, H, I]``
    in e4m3, no expert mask. The reference runs that row through a second weight format (MXFP4 routed + FP8 shared,
    per_1x32 only); here routed and shared experts have the same FP8 block-scale format, so the shared weights are
    copied into the dummy row (four device copies, stream-ordered before the layer) and the row is routed like
    any other expert."""
    if any(t is None for t in shared):
        raise ValueError("shared_w1, shared_w2, shared_w1_scale, and shared_w2_scale must be provided together")
    if quant_type != QuantType.per_1x128:
        raise NotImplementedError("fused_moe: shared_w1/shared_w2 are supported with QuantType.per_1x128 / per_128x128 only")
    if expert_mask is not None:
        raise NotImplementedError("fused_moe: shared expert weights with an expert mask are not supported")
    shared_w1, shared_w2, shared_w1_scale, shared_w2_scale = shared
    E = w1.shape[0]
    if shared_expert_id != E - 1:
        raise ValueError("shared expert weights need a dummy final routed weight row and shared_expert_id == E - 1; "
                         f"got {shared_expert_id=} and E={E}")
    if shared_w1.dtype != dtypes.fp8 or shared_w2.dtype != dtypes.fp8:
        raise ValueError("shared weights must use FP8 E4M3")
    if tuple(shared_w1.shape) != (1, *w1.shape[1:]) or tuple(shared_w2.shape) != (1, *w2.shape[1:]):
        raise ValueError(f"Expected shared_w1 shape {(1, *w1.shape[1:])} and shared_w2 shape {(1, *w2.shape[1:])}, got "
                         f"{tuple(shared_w1.shape)} and {tuple(shared_w2.shape)}")
    for dst, src, name in ((w1, shared_w1, "w1"), (w2, shared_w2, "w2"), (w1_scale, shared_w1_scale, "w1_scale"),
                           (w2_scale, shared_w2_scale, "w2_scale")):
        if not dst.is_contiguous():
            raise ValueError(f"fused_moe: {name} must be contiguous to receive the shared expert's row")
        row = dst.view(E, -1)[E - 1]
        if src.numel() != row.numel():
            raise ValueError(f"shared_{name} has {src.numel()} elements, one expert's {name} has {row.numel()}")
        row.view(torch.uint8).copy_(src.contiguous().view(-1).view(torch.uint8))


def get_inter_dim(w1_shape, w2_shape):
    """aiter/fused_moe.py:448-456."""
    E, _, model_dim = w1_shape
    E, model_dim, inter_dim = w2_shape
    return E, model_dim, inter_dim


# Opt-in kernel-bench hook (the reference's ``kernel_bench_callable``, aiter/fused_moe.py:79-82): a caller sets a
# list here and every layer call appends (name, cuda event) marks before each of its kernels and at its end;
# None in production, so there is no overhead.
kernel_bench_events = None


def _mark(timers, name):
    if timers is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        timers.append((name, ev))


def fused_moe_stages(hidden_states, w1, w2, topk_weight, topk_ids, expert_mask, w1_scale, w2_scale,
                     a1_scale, num_local_tokens, dtype, return_intermediates=False, timers=None,
                     stage2_chunks=1, on_chunk=None, sm_margin=0, quant_type=QuantType.per_1x128,
                     activation=ActivationType.Silu, doweight_stage1=False, stage2_ranges=1):
    """sort -> a1 quant -> stage 1 -> stage 2 -> final rounding (the 2-stage flow of
    aiter/fused_moe.py:2979-3368 with the requant fused into stage 1).

    ``stage2_chunks`` > 1 (with ``dtype=None``) computes the output columns in that many ranges, each into
    its own contiguous fp32 block of the returned [chunks, M, H/chunks] tensor, calling
    ``on_chunk(index, block)`` after each launch so the caller can start a collective on it while the
    next range is computed; ``sm_margin`` SMs are left idle by those launches for the collective's kernels.

    ``stage2_ranges`` > 1 (with ``dtype=None``) also computes the output columns in that many ranges, but into the one
    [M, H] buffer: ``on_chunk(index, (acc, col_begin, col_end))`` is called after each launch, and the launches after the
    first leave ``sm_margin`` SMs idle (the first has nothing running beside it).

    ``timers``: optional list that receives (name, cuda event) marks recorded on the current
    stream before each kernel and at the end (the reference's per-stage bench hook,
    aiter/fused_moe.py:79-82)."""
    device = hidden_states.device
    M, topk = topk_ids.shape
    E, model_dim, inter_dim = get_inter_dim(w1.shape, w2.shape)
    global_E = expert_mask.numel() if expert_mask is not None else E
    if timers is None:
        timers = kernel_bench_events

    _mark(timers, "sort")
    # stage 2 accumulates fp32 sums: the sort's zero-filled moe_buf, asked for as [M, model_dim] fp32, is that
    # accumulator (its spare CTAs clear it beside the scan, so no fill kernel of its own runs); the column-range
    # variant has another layout and clears its own
    sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids, acc_buf = _moe_sorting_impl(
        topk_ids, topk_weight, global_E, model_dim, dtypes.fp32, GEMM_BLOCK_M, expert_mask,
        num_local_tokens, 0, False, want_moe_buf=stage2_chunks == 1)
    if stage2_chunks > 1 and stage2_ranges > 1:
        raise ValueError("stage2_chunks and stage2_ranges exclude each other")
    _mark(timers, "quant")
    # per_Tensor runs through the per_Token kernels: the one activation scale is repeated per row, the one weight
    # scale per expert is repeated per output channel (the reference dequantises both types the same way,
    # aiter/fused_moe.py:3583-3585, 3729-3731)
    per_tensor = QuantType(quant_type) == QuantType.per_Tensor
    per_token = per_tensor or QuantType(quant_type) == QuantType.per_Token
    act = int(ActivationType(activation))
    w_stage1 = sorted_weights if doweight_stage1 else None   # aiter/fused_moe.py:3651-3652
    dw2 = 0 if doweight_stage1 else 1
    qt = int(QuantType.per_Token if per_token else QuantType.per_1x128)
    if hidden_states.dtype == dtypes.fp8:
        a1, a1_s = hidden_states.contiguous(), a1_scale.contiguous().view(M, -1)
    elif per_tensor:
        a1, _scale, a1_s = _per_tensor_quant(hidden_states, want_row_scales=True)
    elif per_token:
        a1, a1_s = per_token_quant_hip(hidden_states, quant_dtype=dtypes.fp8)
    else:
        a1, a1_s = per_group_quant_hip(hidden_states, quant_dtype=dtypes.fp8)

    P = sorted_ids.numel()
    status = _status(device)
    _mark(timers, "stage1")
    if per_token:
        # stage 1 leaves the bf16 activation in sorted-row order; the row scale needs the whole row,
        # so the requantisation is a pass of its own over the valid rows (num_valid_ids[0] on the device)
        a2_bf16 = torch.empty((P, inter_dim), dtype=dtypes.bf16, device=device)
        _lib.call("b200_moe_stage1", a1, a1_s, w1, w1_scale, sorted_ids, sorted_expert_ids, num_valid_ids,
                  a2_bf16, None, status, qt, w_stage1, act, device=device)
        _mark(timers, "requant")
        a2 = torch.empty((P, inter_dim), dtype=dtypes.fp8, device=device)
        a2_s = torch.empty((P,), dtype=dtypes.fp32, device=device)
        if per_tensor:
            _lib.call("b200_moe_quant_per_tensor", a2, a2_bf16, torch.empty((1,), dtype=dtypes.fp32, device=device),
                      torch.empty((1,), dtype=dtypes.fp32, device=device), a2_s, num_valid_ids, device=device)
        else:
            _lib.call("b200_moe_quant_per_token", a2, a2_bf16, a2_s, num_valid_ids, 1, device=device)
    else:
        a2 = torch.empty((P, inter_dim), dtype=dtypes.fp8, device=device)
        a2_s = torch.empty((P, inter_dim // 128), dtype=dtypes.fp32, device=device)
        _lib.call("b200_moe_stage1", a1, a1_s, w1, w1_scale, sorted_ids, sorted_expert_ids, num_valid_ids,
                  a2, a2_s, status, qt, w_stage1, act, device=device)
    _mark(timers, "zero")
    if stage2_chunks > 1:
        if dtype is not None or model_dim % (256 * stage2_chunks) != 0:
            raise ValueError("stage2_chunks needs dtype=None and model_dim divisible by 256*chunks")
        hc = model_dim // stage2_chunks
        acc = torch.zeros((stage2_chunks, M, hc), dtype=dtypes.fp32, device=device)
        _mark(timers, "stage2")
        for c in range(stage2_chunks):
            _lib.call("b200_moe_stage2", a2, a2_s, w2, w2_scale, sorted_ids, sorted_weights, sorted_expert_ids,
                      num_valid_ids, acc[c], status, c * hc, (c + 1) * hc, int(sm_margin), qt, dw2, device=device)
            if on_chunk is not None:
                on_chunk(c, acc[c])
        _mark(timers, "end")
        return acc
    acc = acc_buf
    _mark(timers, "stage2")
    if stage2_ranges > 1:
        if dtype is not None or model_dim % (256 * stage2_ranges) != 0:
            raise ValueError("stage2_ranges needs dtype=None and model_dim divisible by 256*ranges")
        hc = model_dim // stage2_ranges
        for c in range(stage2_ranges):
            _lib.call("b200_moe_stage2", a2, a2_s, w2, w2_scale, sorted_ids, sorted_weights, sorted_expert_ids,
                      num_valid_ids, acc, status, c * hc, (c + 1) * hc, int(sm_margin) if c > 0 else 0, qt, dw2,
                      device=device)
            if on_chunk is not None:
                on_chunk(c, (acc, c * hc, (c + 1) * hc))
        _mark(timers, "end")
        return acc
    _lib.call("b200_moe_stage2", a2, a2_s, w2, w2_scale, sorted_ids, sorted_weights, sorted_expert_ids,
              num_valid_ids, acc, status, 0, 0, 0, qt, dw2, device=device)
    if dtype is None:        # caller wants the fp32 sums (expert parallelism reduces them across ranks first)
        _mark(timers, "end")
        return acc
    _mark(timers, "finalize")
    out = torch.empty((M, model_dim), dtype=dtype, device=device)
    _lib.call("b200_moe_finalize", out, acc, device=device)
    _mark(timers, "end")
    if return_intermediates:
        return out, dict(sorted_ids=sorted_ids, sorted_weights=sorted_weights,
                         sorted_expert_ids=sorted_expert_ids, num_valid_ids=num_valid_ids,
                         a1=a1, a1_scale=a1_s, a2=a2, a2_scale=a2_s, acc=acc)
    return out


def fused_moe(
    hidden_states,
    w1,  # [expert(local_expert:EP), inter_dim*2, dim] N,K
    w2,  # [expert(local_expert:EP), dim, inter_dim]
    topk_weight,
    topk_ids,
    expert_mask=None,  # EP
    activation=ActivationType.Silu,
    quant_type=QuantType.No,
    doweight_stage1=False,
    # following for quant
    w1_scale=None,  # [expert, 2*inter_dim/128, dim/128] (or any shape with that many elements)
    w2_scale=None,  # [expert, dim/128, inter_dim/128]
    a1_scale=None,  # [tokens, dim/128] when hidden_states is already fp8
    a2_scale=None,
    # following for tuning
    block_size_M=None,
    num_local_tokens=None,
    moe_sorting_dispatch_policy=0,
    dtype=None,
    # following for cktile support
    hidden_pad=0,
    intermediate_pad=0,
    bias1=None,
    bias2=None,
    splitk=0,
    swiglu_limit=None,
    beta=None,
    linear_beta=None,
    gate_mode="separated",
    shared_w1=None,
    shared_w2=None,
    shared_w1_scale=None,
    shared_w2_scale=None,
    shared_expert_id=-1,
    stage2_scatter=None,
):
    """Drop-in for aiter.fused_moe (aiter/fused_moe.py:458-576) on the FP8 block-scale path.

    hidden_states [M, H] bf16 (or e4m3 + a1_scale [M, H/128]); w1 [E, 2I, H] e4m3, gate rows then
    up rows; w2 [E, H, I] e4m3; w1_scale/w2_scale fp32 per 128x128 block; topk_weight [M, topk]
    fp32; topk_ids [M, topk] int32 (global expert ids when expert_mask is given).  Returns [M, H]
    in ``dtype`` (default: hidden_states.dtype; bf16 when that is fp8).

    ``block_size_M`` is accepted and ignored: the GEMM row tile is fixed at 128, which only
    changes how the routes are padded, not the result.

    The call only enqueues work. Should a device-side wait of a GEMM kernel ever run out (a broken pipeline; the
    kernels then stop by themselves instead of hanging the GPU), the output is incomplete and a per-device status word
    is set: call ``check_device_status()`` after synchronising to learn of it (it raises and clears the word). The word
    is shared by all streams of a device. Setting ``AITER_B200_CHECK_STATUS=1`` makes every layer call check it (one
    host synchronisation per call: a debugging aid, not for serving)."""
    quant_type = quant_remap.get(QuantType(quant_type), QuantType(quant_type))
    if quant_type not in (QuantType.per_1x128, QuantType.per_Token, QuantType.per_Tensor):
        raise NotImplementedError(
            f"fused_moe: quant_type={QuantType(quant_type)!r} is not supported; this build covers "
            "QuantType.per_1x128 / per_128x128 (FP8 block scale), QuantType.per_Token and QuantType.per_Tensor (FP8)")
    if ActivationType(activation) not in (ActivationType.Silu, ActivationType.Gelu):
        raise NotImplementedError(f"fused_moe: activation={ActivationType(activation)!r} is not supported (Silu, Gelu)")
    _check_unsupported(
        a2_scale=(a2_scale, None),
        hidden_pad=(hidden_pad, 0), intermediate_pad=(intermediate_pad, 0), bias1=(bias1, None),
        bias2=(bias2, None), splitk=(splitk or 0, 0), swiglu_limit=(swiglu_limit, None),
        beta=(beta, None), linear_beta=(linear_beta, None), stage2_scatter=(stage2_scatter, None))
    if gate_mode not in (None, "separated"):
        raise NotImplementedError(f"fused_moe: gate_mode={gate_mode!r} is not supported (separated only)")
    if not hidden_states.is_cuda:
        raise RuntimeError("fused_moe: tensors must live on a CUDA device (there is no CPU path)")
    if w1.dtype != dtypes.fp8 or w2.dtype != dtypes.fp8:
        raise NotImplementedError(f"fused_moe: weights must be float8_e4m3fn, got {w1.dtype}/{w2.dtype}")
    if w1_scale is None or w2_scale is None:
        raise ValueError("fused_moe: w1_scale and w2_scale are required for FP8 quantisation")
    M, topk = topk_ids.shape
    E, model_dim, inter_dim = get_inter_dim(w1.shape, w2.shape)
    if w1.shape[1] != 2 * inter_dim:
        raise NotImplementedError(f"fused_moe: only gated (g1u1) weights are supported: {w1.shape=} {w2.shape=}")
    if inter_dim % 128 != 0 or model_dim % 128 != 0:
        # csrc/py_itfs_cu/asm_fmoe.cu:926, gemm_moe_ck2stages_common_blockscale.cuh:106-108
        raise ValueError(f"fused_moe: inter_dim ({inter_dim}) and model_dim ({model_dim}) must be multiples of 128")
    if hidden_states.shape != (M, model_dim):
        raise ValueError(f"fused_moe: hidden_states must be [{M}, {model_dim}], got {tuple(hidden_states.shape)}")
    if hidden_states.dtype == dtypes.fp8:
        if a1_scale is None:
            raise ValueError("fused_moe: fp8 hidden_states need a1_scale ([M, model_dim/128], or [M, 1] for per_Token)")
        dtype = dtypes.bf16 if dtype is None else dtype
    else:
        if hidden_states.dtype not in (dtypes.bf16, dtypes.fp16):   # aiter/fused_moe.py:752-756
            raise NotImplementedError(f"fused_moe: hidden_states must be bf16, fp16 or pre-quantised fp8, got {hidden_states.dtype}")
        if a1_scale is not None:
            raise NotImplementedError("fused_moe: a1_scale with un-quantised hidden_states is not supported")
        dtype = hidden_states.dtype if dtype is None else dtype
    # aiter/fused_moe.py:752-756
    assert dtype in [dtypes.fp16, dtypes.bf16], f"Fused_moe unsupported out dtype: {dtype}"
    if topk_weight.dtype != dtypes.fp32:
        raise ValueError("fused_moe: topk_weight must be float32")
    if topk_ids.dtype != dtypes.i32:
        raise ValueError("fused_moe: topk_ids must be int32")
    if quant_type == QuantType.per_Tensor:
        if hidden_states.dtype == dtypes.fp8:
            a1_scale = a1_scale.to(dtypes.fp32).reshape(-1)[:1].expand(M).contiguous()
        # one scale per expert -> one per output channel, the layout the per_Token kernels read
        w1_scale = w1_scale.to(dtypes.fp32).reshape(E, 1).expand(E, 2 * inter_dim)
        w2_scale = w2_scale.to(dtypes.fp32).reshape(E, 1).expand(E, model_dim)
    shared = (shared_w1, shared_w2, shared_w1_scale, shared_w2_scale)
    if any(t is not None for t in shared) or shared_expert_id != -1:
        _fold_shared_expert(w1, w2, w1_scale, w2_scale, shared, shared_expert_id, quant_type, expert_mask)
    if M == 0:   # nothing to compute: the reference allocates the same empty result (aiter/fused_moe.py:579-619)
        return torch.empty((0, model_dim), dtype=dtype, device=hidden_states.device)
    out = fused_moe_stages(hidden_states, w1.contiguous(), w2.contiguous(), topk_weight, topk_ids,
                           expert_mask, w1_scale.contiguous(), w2_scale.contiguous(), a1_scale,
                           num_local_tokens, dtype, quant_type=quant_type, activation=activation,
                           doweight_stage1=bool(doweight_stage1))
    if _CHECK_STATUS_EVERY_CALL:
        check_device_status(hidden_states.device)
    return out


# ------------------------------------------------------------------------------------- torch integration
def shuffle_weight(x, layout=(16, 16), use_int4=False, is_guinterleave=False, gate_up=False, pad_k_to=0):
    """Weight prepack hook with the signature of aiter/ops/shuffle.py:148-209.

    The reference permutes weights into 16x16 MFMA tiles and marks them ``is_shuffled``; on B200 the
    TMA reads the plain K-major ``[E, N, K]`` rows, so the prepack is the identity. The attribute
    protocol is kept (``fused_moe`` in the reference reads it, aiter/fused_moe.py:747) so loaders that
    call ``shuffle_weight`` once at model load keep working."""
    if use_int4 or is_guinterleave or pad_k_to:
        raise NotImplementedError("shuffle_weight: int4 / gate-up interleave / K padding are not supported")
    x.is_shuffled = True
    return x


def _fused_moe_fake(hidden_states, w1, w2, topk_weight, topk_ids, expert_mask=None, activation=0, quant_type=0,
                    doweight_stage1=False, w1_scale=None, w2_scale=None, a1_scale=None, num_local_tokens=None,
                    dtype=None):
    """Shape/dtype propagation of aiter/fused_moe.py:579-619: empty((M, model_dim), dtype)."""
    M = topk_ids.shape[0]
    out_dtype = dtype if dtype is not None else (dtypes.bf16 if hidden_states.dtype == dtypes.fp8 else hidden_states.dtype)
    return torch.empty((M, w2.shape[1]), dtype=out_dtype, device=topk_ids.device)


@torch.library.custom_op("aiter_b200::fused_moe_", mutates_args=(), device_types="cuda")
def fused_moe_(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weight: torch.Tensor,
               topk_ids: torch.Tensor, expert_mask: torch.Tensor | None = None, activation: int = 0,
               quant_type: int = 0, doweight_stage1: bool = False, w1_scale: torch.Tensor | None = None,
               w2_scale: torch.Tensor | None = None, a1_scale: torch.Tensor | None = None,
               num_local_tokens: torch.Tensor | None = None, dtype: torch.dtype | None = None) -> torch.Tensor:
    """The layer as a registered torch operator (enums as ints, like the reference's ``fused_moe_``,
    aiter/fused_moe.py:622-695), so that graphs traced by torch.compile carry it as one opaque call."""
    return fused_moe(hidden_states, w1, w2, topk_weight, topk_ids, expert_mask=expert_mask,
                     activation=ActivationType(activation), quant_type=QuantType(quant_type),
                     doweight_stage1=doweight_stage1, w1_scale=w1_scale, w2_scale=w2_scale, a1_scale=a1_scale,
                     num_local_tokens=num_local_tokens, dtype=dtype)


fused_moe_.register_fake(_fused_moe_fake)
