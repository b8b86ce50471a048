"""Generates the fixtures in this directory from the UNMODIFIED reference functions.

Needs a checkout of ROCm/aiter (its path in ``AITER_REFERENCE_ROOT``; ``oracle/ref_loader.py`` holds the default); it
cannot run on a machine without one, which is why its outputs are committed.  For every
case it also runs the restatement in ``oracle/moe_oracle.py`` on the same inputs and
asserts bit-identity, so a fixture is only ever written from a pinned oracle.

    python tests/golden/make_golden.py

Fixtures (numpy ``.npz``; bf16 stored as its uint16 bit pattern, e4m3 as uint8):
  sorting_kat.npz     worked example of csrc/include/moe_sorting_opus.h:284-346 and the
                      3x3 known-answer case of op_tests/test_moe_local_expert_ids.py:13-63
  sorting_sweep.npz   run_torch_moe_sorting on seeded random routings
  quant_1x128.npz     pertoken_quant on seeded rows with edge groups
  cfg0.npz            torch_moe_stage1/2 pipeline on the tiny layer (M=32,H=1024,I=512,E=8,topk=2)
  cfg0_ep2.npz        the same layer split over 2 expert-parallel ranks (local ids + mask)
  dsv3_slice.npz      DeepSeek-V3 dimensions with 8 experts (M=16,H=7168,I=2048,topk=8)
  cfg0_per_token.npz  the tiny layer with QuantType.per_Token (row scales, per-output-channel weight scales)
  cfg0_per_tensor.npz the tiny layer with QuantType.per_Tensor (one activation scale, one weight scale per expert)
  cfg0_variants.npz   the tiny layer with Gelu and/or doweight_stage1
  routing_dsv3.npz    biased_grouped_topk_torch (8 groups, top-4 groups, top-8, x2.5)
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import inputs, moe_oracle, ref_loader  # noqa: E402

FP8 = torch.float8_e4m3fn


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == FP8:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def same(a, b):
    return a.shape == b.shape and np.array_equal(bits(a), bits(b))


def save(name, **arrays):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"wrote {name}: {os.path.getsize(path) / 1024:.1f} KiB")


def ref_pipeline(ref, x, w1_q, w1_s, w2_q, w2_s, tw, ids):
    """op_tests/test_moe_2stage.py per_128x128 branch, through the reference functions."""
    M, H = x.shape
    topk = ids.shape[1]
    QT = ref.QuantType.per_128x128
    a1_q, a1_s = ref.pertoken_quant(x.view(M, -1, 128), quant_dtype=FP8)
    a1_q = a1_q.view(M, H)
    a1_s = a1_s.squeeze(-1)
    out1 = ref.torch_moe_stage1(a1_q, w1_q, w2_q, tw, ids, dtype=torch.bfloat16,
                                activation=ref.ActivationType.Silu, quant_type=QT,
                                a1_scale=a1_s, w1_scale=w1_s)
    a2_q, a2_s = ref.pertoken_quant(out1.view(M, -1, 128), quant_dtype=FP8)
    a2_q = a2_q.view(M, topk, -1)
    a2_s = a2_s.view(M, topk, -1)
    out = ref.torch_moe_stage2(a2_q, w1_q, w2_q, tw, ids, dtype=torch.bfloat16, quant_type=QT,
                               w2_scale=w2_s, a2_scale=a2_s)
    return dict(a1_q=a1_q, a1_scale=a1_s, out1=out1, a2_q=a2_q, a2_scale=a2_s, out=out)


def ref_pipeline_per_token(ref, x, w1_q, w1_s, w2_q, w2_s, tw, ids):
    """op_tests/test_moe_2stage.py, QuantType.per_Token branch (:213-214, :264, :397-460)."""
    M, H = x.shape
    topk = ids.shape[1]
    QT = ref.QuantType.per_Token
    a1_q, a1_s = ref.pertoken_quant(x, quant_dtype=FP8)
    out1 = ref.torch_moe_stage1(a1_q, w1_q, w2_q, tw, ids, dtype=torch.bfloat16,
                                activation=ref.ActivationType.Silu, quant_type=QT,
                                a1_scale=a1_s, w1_scale=w1_s)
    a2_q, a2_s = ref.pertoken_quant(out1, quant_dtype=FP8)
    a2_q = a2_q.view(M, topk, -1)
    out = ref.torch_moe_stage2(a2_q, w1_q, w2_q, tw, ids, dtype=torch.bfloat16, quant_type=QT,
                               w2_scale=w2_s, a2_scale=a2_s)
    return dict(a1_q=a1_q, a1_scale=a1_s, out1=out1, a2_q=a2_q, a2_scale=a2_s, out=out)


def ref_pipeline_per_tensor(ref, x, w1_q, w1_s, w2_q, w2_s, tw, ids):
    """op_tests/test_moe_2stage.py, QuantType.per_Tensor branch (:160-164 weights, torch_quant = per_tensor_quant for
    the activations :264, :446)."""
    M, H = x.shape
    topk = ids.shape[1]
    QT = ref.QuantType.per_Tensor
    a1_q, a1_s = ref.per_tensor_quant(x, quant_dtype=FP8)
    out1 = ref.torch_moe_stage1(a1_q, w1_q, w2_q, tw, ids, dtype=torch.bfloat16,
                                activation=ref.ActivationType.Silu, quant_type=QT,
                                a1_scale=a1_s, w1_scale=w1_s)
    a2_q, a2_s = ref.per_tensor_quant(out1, quant_dtype=FP8)
    a2_q = a2_q.view(M, topk, -1)
    out = ref.torch_moe_stage2(a2_q, w1_q, w2_q, tw, ids, dtype=torch.bfloat16, quant_type=QT,
                               w2_scale=w2_s, a2_scale=a2_s)
    return dict(a1_q=a1_q, a1_scale=a1_s, out1=out1, a2_q=a2_q, a2_scale=a2_s, out=out)


def layer_case(ref, name, fname):
    c = inputs.make_config(name, seed=0)
    pt = c["cfg"].get("quant") == "per_token"
    pten = c["cfg"].get("quant") == "per_tensor"
    pipe = ref_pipeline_per_tensor if pten else ref_pipeline_per_token if pt else ref_pipeline
    r = pipe(ref, c["x"], c["w1_q"], c["w1_scale"], c["w2_q"], c["w2_scale"],
             c["topk_weight"], c["topk_ids"])
    out, st = moe_oracle.fused_moe_ref(c["x"], c["w1_q"], c["w1_scale"], c["w2_q"], c["w2_scale"],
                                       c["topk_weight"], c["topk_ids"], return_stages=True, per_token=pt,
                                       per_tensor=pten)
    if pt:
        st = dict(st, a1_scale=st["a1_scale"].view(r["a1_scale"].shape), a2_scale=st["a2_scale"].view(r["a2_scale"].shape))
    for k in ("a1_q", "a1_scale", "out1", "a2_q", "a2_scale"):
        assert same(r[k], st[k]), f"{name}: restatement differs from reference at {k}"
    assert same(r["out"], out), f"{name}: restatement differs from reference at out"
    save(fname, topk_ids=bits(c["topk_ids"]), topk_weight=bits(c["topk_weight"]),
         x_sum=np.float64(c["x"].double().sum()),
         w1_scale=bits(c["w1_scale"]), w2_scale=bits(c["w2_scale"]),
         w1_q_sum=np.int64(c["w1_q"].view(torch.uint8).long().sum()),
         w2_q_sum=np.int64(c["w2_q"].view(torch.uint8).long().sum()),
         a1_q=bits(r["a1_q"]), a1_scale=bits(r["a1_scale"]), out1=bits(r["out1"]),
         a2_q=bits(r["a2_q"]), a2_scale=bits(r["a2_scale"]), out=bits(r["out"]))
    return c, r


def main():
    assert ref_loader.available(), "reference checkout not found"
    ref = ref_loader.load()
    torch.manual_seed(0)

    # ---- sorting: known answers --------------------------------------------------------
    ids = torch.tensor([[0, 3, 5], [2, 3, 5], [1, 3, 5], [1, 2, 3], [1, 3, 5]], dtype=torch.int32)
    w = torch.arange(1, 16, dtype=torch.float32).view(5, 3) / 16
    mask = torch.tensor([1, 0, 1, 1, 0, 1], dtype=torch.int32)
    kat = {}
    for tag, m in (("plain", None), ("masked", mask)):
        r = ref.run_torch_moe_sorting(ids, w, 6, 4, m, None)
        o = moe_oracle.moe_sorting_ref(ids, w, 6, 4, m, None)
        n = int(r[3][0])
        assert same(r[0][:n], o[0][:n]) and same(r[2], o[2]) and same(r[3], o[3])
        pad = r[0][:n] == (3 << 24 | 5)
        assert same(r[1][:n][~pad], o[1][:n][~pad])
        kat.update({f"{tag}_sorted_ids": bits(o[0]), f"{tag}_sorted_weights": bits(o[1]),
                    f"{tag}_sorted_expert_ids": bits(o[2]), f"{tag}_num_valid": bits(o[3])})
    # values stated in the header comment: 24 slots / [0,1,2,3,3,5]; masked 20 / [0,1,2,2,3]
    assert int(kat["plain_num_valid"][0]) == 24 and list(kat["plain_sorted_expert_ids"][:6]) == [0, 1, 2, 3, 3, 5]
    assert int(kat["masked_num_valid"][0]) == 20 and list(kat["masked_sorted_expert_ids"][:5]) == [0, 1, 2, 2, 3]
    # op_tests/test_moe_local_expert_ids.py:13-63
    ids3 = torch.tensor([[0, 1, 5], [2, 4, 3], [5, 0, 2]], dtype=torch.int32)
    mask3 = torch.tensor([0, 1, 1, 0, 1, 0], dtype=torch.int32)
    local = moe_oracle.local_expert_ids(ids3, mask3)
    assert local.tolist() == [[-1, 0, -1], [1, 2, -1], [-1, -1, 1]]
    save("sorting_kat.npz", topk_ids=bits(ids), topk_weights=bits(w), mask=bits(mask),
         ids3=bits(ids3), mask3=bits(mask3), local3=bits(local), **kat)

    # ---- sorting: seeded sweep ----------------------------------------------------------
    sweep = {}
    cases = [(1, 32, 5, 32), (7, 8, 2, 16), (33, 40, 6, 32), (128, 256, 8, 128),
             (777, 385, 7, 64), (2048, 256, 8, 128), (64, 256, 8, 128)]
    for ci, (M, E, topk, B) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + ci)
        sc = torch.rand((M, E), generator=g)
        tw, ti = torch.topk(sc, topk, dim=-1)
        ti = ti.to(torch.int32)
        for tag, m, nl in (("a", None, None),
                           ("b", (torch.rand(E, generator=g) > 0.5).to(torch.int32), None),
                           ("c", None, torch.tensor([max(1, M // 2)], dtype=torch.int32))):
            r = ref.run_torch_moe_sorting(ti, tw, E, B, m, nl)
            o = moe_oracle.moe_sorting_ref(ti, tw, E, B, m, nl)
            n = int(r[3][0])
            assert same(r[0], o[0]) and same(r[2], o[2]) and same(r[3], o[3])
            pad = r[0][:n] == (topk << 24 | M)
            assert same(r[1][:n][~pad], o[1][:n][~pad])
            key = f"c{ci}{tag}"
            sweep[key + "_meta"] = np.array([M, E, topk, B, 100 + ci], dtype=np.int64)
            sweep[key + "_ids"] = bits(ti)
            sweep[key + "_w"] = bits(tw)
            if m is not None:
                sweep[key + "_mask"] = bits(m)
            if nl is not None:
                sweep[key + "_nl"] = bits(nl)
            sweep[key + "_sorted_ids"] = bits(o[0])
            sweep[key + "_sorted_weights"] = bits(o[1])
            sweep[key + "_sorted_expert_ids"] = bits(o[2])
            sweep[key + "_num_valid"] = bits(o[3])
    save("sorting_sweep.npz", **sweep)

    # ---- 1x128 quant --------------------------------------------------------------------
    g = torch.Generator().manual_seed(7)
    xq = (torch.randn((48, 1024), generator=g) * 3).to(torch.bfloat16)
    xq[0, :128] = 0                       # all-zero group -> scale 1
    xq[1, 128:256] = 448.0                # amax exactly at the fp8 max
    xq[2, :128] = 1e-30                   # flushes to 0 in bf16? (kept as is)
    xq[3, 256:384] *= 1e4                 # large dynamic range
    xq[4, :128] = torch.linspace(-1, 1, 128).to(torch.bfloat16)
    q_r, s_r = ref.pertoken_quant(xq.view(48, -1, 128), quant_dtype=FP8)
    q_o, s_o = moe_oracle.quant_1x128(xq)
    assert same(q_r.view(48, 1024), q_o) and same(s_r.squeeze(-1), s_o)
    save("quant_1x128.npz", x=bits(xq), q=bits(q_o), scale=bits(s_o))

    # ---- full layers --------------------------------------------------------------------
    c0, r0 = layer_case(ref, "cfg0", "cfg0.npz")
    layer_case(ref, "dsv3_slice", "dsv3_slice.npz")
    layer_case(ref, "cfg0_pt", "cfg0_per_token.npz")
    layer_case(ref, "cfg0_ptensor", "cfg0_per_tensor.npz")

    # ---- activation / weighting variants on the tiny layer (aiter/fused_moe.py:3651-3652, 3665-3681) ----
    var = {}
    for tag, act_ref, act, dw1 in (("gelu", ref.ActivationType.Gelu, "gelu", False),
                                   ("doweight1", ref.ActivationType.Silu, "silu", True),
                                   ("gelu_doweight1", ref.ActivationType.Gelu, "gelu", True)):
        QT = ref.QuantType.per_128x128
        M, topk = c0["topk_ids"].shape
        o1 = ref.torch_moe_stage1(r0["a1_q"], c0["w1_q"], c0["w2_q"], c0["topk_weight"], c0["topk_ids"],
                                  dtype=torch.bfloat16, activation=act_ref, quant_type=QT, a1_scale=r0["a1_scale"],
                                  w1_scale=c0["w1_scale"], doweight=dw1)
        q2, s2 = ref.pertoken_quant(o1.view(M, -1, 128), quant_dtype=FP8)
        o = ref.torch_moe_stage2(q2.view(M, topk, -1), c0["w1_q"], c0["w2_q"], c0["topk_weight"], c0["topk_ids"],
                                 dtype=torch.bfloat16, quant_type=QT, w2_scale=c0["w2_scale"],
                                 a2_scale=s2.view(M, topk, -1), doweight=not dw1)
        mine = moe_oracle.fused_moe_ref(c0["x"], c0["w1_q"], c0["w1_scale"], c0["w2_q"], c0["w2_scale"],
                                        c0["topk_weight"], c0["topk_ids"], activation=act, doweight_stage1=dw1)
        assert same(o, mine), tag
        var[tag] = bits(o)
    save("cfg0_variants.npz", **var)

    # ---- expert parallel, 2 ranks (masking as in aiter/fused_moe.py:3467-3470) -----------
    E = c0["cfg"]["E"]
    ep = {}
    total = torch.zeros(r0["out"].shape, dtype=torch.float32)
    for rank in range(2):
        m = torch.zeros(E, dtype=torch.int32)
        m[rank * E // 2:(rank + 1) * E // 2] = 1
        sl = slice(rank * E // 2, (rank + 1) * E // 2)
        local = moe_oracle.local_expert_ids(c0["topk_ids"], m)
        r = ref_pipeline(ref, c0["x"], c0["w1_q"][sl], c0["w1_scale"][sl], c0["w2_q"][sl],
                         c0["w2_scale"][sl], c0["topk_weight"], local)
        o = moe_oracle.fused_moe_ref(c0["x"], c0["w1_q"][sl], c0["w1_scale"][sl], c0["w2_q"][sl],
                                     c0["w2_scale"][sl], c0["topk_weight"], c0["topk_ids"],
                                     expert_mask=m)
        assert same(r["out"], o)
        ep[f"mask{rank}"] = bits(m)
        ep[f"out{rank}"] = bits(o)
        total += o.float()
    ep["sum_bf16"] = bits(total.to(torch.bfloat16))
    save("cfg0_ep2.npz", **ep)

    # ---- DeepSeek-V3 routing ------------------------------------------------------------
    g = torch.Generator().manual_seed(11)
    logits = torch.randn((64, 256), generator=g)
    bias = torch.randn((256,), generator=g) * 0.1
    w_r, i_r = ref.biased_grouped_topk_torch(logits, bias, 8, True, 8, 4)
    w_o, i_o = moe_oracle.biased_grouped_topk_ref(logits, bias, 8, True, 8, 4, 1.0)
    assert same(w_r, w_o) and same(i_r, i_o)
    w_o, i_o = moe_oracle.biased_grouped_topk_ref(logits, bias, 8, True, 8, 4, 2.5)
    save("routing_dsv3.npz", logits=bits(logits), bias=bits(bias), weights=bits(w_o), ids=bits(i_o))
    print("all fixtures pinned against the reference")


if __name__ == "__main__":
    main()
