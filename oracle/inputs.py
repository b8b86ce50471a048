"""Seeded synthetic inputs for the benchmark configurations (test infrastructure only).

The reference's tests draw fresh ``torch.randn`` tensors (op_tests/test_moe_2stage.py:108-123)
and quantise them with ``weight_per_128x128_quant`` (:184-208); there is no dataset.  The
configurations below keep those distributions with the shapes of the five benchmark cases.
Weights are generated and quantised one expert at a time so a DeepSeek-V3 sized layer
(11.3 GB of e4m3 codes) never needs its bf16/fp32 form resident.
"""

from __future__ import annotations

import math

import torch

from .moe_oracle import (FP8, biased_grouped_topk_ref, quant_per_token, quant_weight_128x128,
                         softmax_topk_ref)

# per_Tensor weights: one scale per expert (op_tests/test_moe_2stage.py:160-164, pertoken_quant over w.view(E, -1))

# name -> dict(M, H, I, E, topk, routing)
CONFIGS = {
    # tiny layer the reference's torch oracle runs on CPU
    "cfg0": dict(M=32, H=1024, I=512, E=8, topk=2, routing="softmax"),
    # DeepSeek-V3 shaped, decode
    "cfg1": dict(M=64, H=7168, I=2048, E=256, topk=8, routing="dsv3"),
    # DeepSeek-V3 shaped, prefill
    "cfg2": dict(M=8192, H=7168, I=2048, E=256, topk=8, routing="dsv3"),
    # Mixtral-8x7B shaped
    "cfg3": dict(M=4096, H=4096, I=14336, E=8, topk=2, routing="softmax", quant="per_token"),
    # the tiny layer with per-token activation scales and per-output-channel weight scales
    "cfg0_pt": dict(M=32, H=1024, I=512, E=8, topk=2, routing="softmax", quant="per_token"),
    # the tiny layer with one activation scale per tensor and one weight scale per expert
    "cfg0_ptensor": dict(M=32, H=1024, I=512, E=8, topk=2, routing="softmax", quant="per_tensor"),
    # Qwen3-235B-A22B shaped, skewed routing (M is swept by the caller)
    "cfg4": dict(M=1024, H=4096, I=1536, E=128, topk=8, routing="zipf"),
    # DeepSeek-V3 dimensions with few experts: cheap enough for CPU goldens
    "dsv3_slice": dict(M=16, H=7168, I=2048, E=8, topk=8, routing="softmax"),
}


def _gen(seed: int, device="cpu"):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_routing(kind, M, E, topk, seed, device="cpu"):
    """Router outputs (fp32 weights [M,topk], int32 ids [M,topk])."""
    g = _gen(seed + 3)
    logits = torch.randn((M, E), generator=g, dtype=torch.float32)
    if kind == "softmax":
        w, ids = softmax_topk_ref(logits, topk, renormalize=True)
    elif kind == "dsv3":
        bias = torch.randn((E,), generator=g, dtype=torch.float32) * 0.1
        w, ids = biased_grouped_topk_ref(logits, bias, topk, True, 8, 4,
                                         routed_scaling_factor=2.5)
    elif kind == "zipf":
        # 8 distinct experts per token from Zipf(s=1.2) over a seeded permutation of
        # expert ids; weights = softmax of N(0,1) over the chosen experts.
        perm = torch.randperm(E, generator=g)
        p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** 1.2
        p = (p / p.sum()).to(torch.float32)
        ranks = torch.multinomial(p.expand(M, E), topk, replacement=False, generator=g)
        ids = perm[ranks].to(torch.int32)
        w = torch.softmax(torch.randn((M, topk), generator=g, dtype=torch.float32), dim=-1)
    else:
        raise ValueError(kind)
    return w.to(device), ids.to(device)


def make_weights(E, N, K, seed, device="cpu", experts_per_chunk=1, per_token=False, per_tensor=False):
    """[E,N,K] ~ N(0, 1/sqrt(K)) quantised to e4m3 per 128x128 block with
    scale = amax/448 (op_tests/test_moe_2stage.py:184-208), or per output channel
    (scales [E,N,1]) for QuantType.per_Token (:213-214)."""
    g = _gen(seed, device)
    q = torch.empty((E, N, K), dtype=FP8, device=device)
    s = (torch.empty((E, 1), dtype=torch.float32, device=device) if per_tensor else
         torch.empty((E, N, 1), dtype=torch.float32, device=device) if per_token else
         torch.empty((E, N // 128, K // 128), dtype=torch.float32, device=device))
    std = 1.0 / math.sqrt(K)
    for e0 in range(0, E, experts_per_chunk):
        e1 = min(E, e0 + experts_per_chunk)
        w = torch.randn((e1 - e0, N, K), generator=g, dtype=torch.float32, device=device) * std
        if per_tensor:
            qe, se = quant_per_token(w.view(e1 - e0, -1))
            qe = qe.view(e1 - e0, N, K)
        else:
            qe, se = quant_per_token(w) if per_token else quant_weight_128x128(w)
        q[e0:e1] = qe
        s[e0:e1] = se
    return q, s


def make_config(name, seed=0, device="cpu", M=None, E=None, weights=None):
    """Returns dict(x bf16 [M,H], w1_q, w1_scale, w2_q, w2_scale, topk_weight, topk_ids, cfg).

    ``x`` and the routing are always drawn on the CPU generator (so goldens do not depend on
    the device); ``device`` only selects where the (large) weights are drawn and quantised. ``weights`` = the
    (w1_q, w1_scale, w2_q, w2_scale) of an earlier call with the same seed, shapes and quantisation is reused
    instead of being drawn again (the DeepSeek-V3 cases share 11.3 GB of them)."""
    cfg = dict(CONFIGS[name])
    if M is not None:
        cfg["M"] = M
    if E is not None:
        cfg["E"] = E
    M_, H, I, E_, topk = cfg["M"], cfg["H"], cfg["I"], cfg["E"], cfg["topk"]
    x = torch.randn((M_, H), generator=_gen(seed), dtype=torch.float32).to(torch.bfloat16)
    pt, pten = cfg.get("quant") == "per_token", cfg.get("quant") == "per_tensor"
    if weights is not None:
        w1_q, w1_s, w2_q, w2_s = weights
        assert tuple(w1_q.shape) == (E_, 2 * I, H) and tuple(w2_q.shape) == (E_, H, I)
    else:
        w1_q, w1_s = make_weights(E_, 2 * I, H, seed + 1, device, per_token=pt, per_tensor=pten)
        w2_q, w2_s = make_weights(E_, H, I, seed + 2, device, per_token=pt, per_tensor=pten)
    tw, ti = make_routing(cfg["routing"], M_, E_, topk, seed)
    return dict(x=x.to(device), w1_q=w1_q, w1_scale=w1_s, w2_q=w2_q, w2_scale=w2_s,
                topk_weight=tw.to(device), topk_ids=ti.to(device), cfg=cfg)
