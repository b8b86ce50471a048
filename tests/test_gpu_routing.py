"""Router kernels against the reference's torch functions (fixture + live oracle).

Expert sets must match; the order inside a token's top-k is not part of the contract (the reference's
own test compares order-insensitively, op_tests/test_moeTopkSoftmax.py:262-376). Two experts whose scores
differ by less than an fp32 ulp of the sigmoid/softmax may swap; such tokens are counted and bounded."""

import numpy as np
import pytest
import torch

from conftest import load_golden

import aiter_b200
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def compare(w, ids, w_ref, ids_ref, tag):
    w, ids = w.cpu(), ids.cpu().long()
    ids_ref = ids_ref.long()
    so, sr = ids.sort(dim=1), ids_ref.sort(dim=1)
    same = (so.values == sr.values).all(dim=1)
    if not bool(same.all()):
        # a different set is only legitimate where experts tie (bf16 logits tie often): the selected
        # weights, as sorted lists, must then still agree
        wa = w[~same].sort(dim=1).values
        wb = w_ref[~same].sort(dim=1).values
        assert torch.allclose(wa, wb, rtol=2e-6, atol=1e-7), f"{tag}: expert sets differ on {int((~same).sum())} tokens"
        assert float(same.float().mean()) >= 0.98, f"{tag}: too many tied tokens ({int((~same).sum())})"
    wo = torch.gather(w, 1, so.indices)[same]
    wr = torch.gather(w_ref, 1, sr.indices)[same]
    assert torch.allclose(wo, wr, rtol=2e-6, atol=1e-7), f"{tag}: weights differ by {float((wo - wr).abs().max())}"
    assert all(len(set(r.tolist())) == ids.shape[1] for r in ids[:64]), "duplicate experts in a token's top-k"


def test_dsv3_routing_fixture():
    g = load_golden("routing_dsv3.npz")
    logits, bias = torch.from_numpy(g["logits"]), torch.from_numpy(g["bias"])
    w = torch.empty((64, 8), dtype=torch.float32, device=DEV)
    ids = torch.empty((64, 8), dtype=torch.int32, device=DEV)
    aiter_b200.biased_grouped_topk(logits.to(DEV), bias.to(DEV), w, ids, 8, 4, True, 2.5)
    compare(w, ids, torch.from_numpy(g["weights"]), torch.from_numpy(g["ids"]), "fixture")
    # the routing feeds the sort unchanged: every token's experts come from at most 4 groups of 32
    assert all(len(set((r // 32).tolist())) <= 4 for r in ids.cpu())


@pytest.mark.parametrize("M,E,topk,groups,topk_group,renorm,scale,dtype", [
    (1, 256, 8, 8, 4, True, 2.5, torch.float32), (777, 256, 8, 8, 4, True, 2.5, torch.bfloat16),
    (300, 128, 6, 8, 3, False, 1.0, torch.float32), (64, 64, 4, 4, 2, True, 1.0, torch.float32),
    (129, 384, 8, 8, 4, True, 2.5, torch.float32), (33, 32, 2, 1, 1, True, 1.0, torch.float32),
])
def test_biased_grouped_topk_against_oracle(M, E, topk, groups, topk_group, renorm, scale, dtype):
    g = torch.Generator().manual_seed(M * 7 + E)
    logits = torch.randn((M, E), generator=g).to(dtype)
    bias = torch.randn((E,), generator=g) * 0.1
    w_ref, ids_ref = moe_oracle.biased_grouped_topk_ref(logits, bias, topk, renorm, groups, topk_group, scale)
    w = torch.empty((M, topk), dtype=torch.float32, device=DEV)
    ids = torch.empty((M, topk), dtype=torch.int32, device=DEV)
    aiter_b200.biased_grouped_topk(logits.to(DEV), bias.to(DEV), w, ids, groups, topk_group, renorm, scale)
    compare(w, ids, w_ref, ids_ref, f"{M}x{E} top{topk}")


@pytest.mark.parametrize("M,E,topk,renorm,dtype", [
    (1, 8, 2, True, torch.float32), (4096, 8, 2, True, torch.bfloat16), (257, 128, 8, True, torch.float32),
    (100, 60, 5, False, torch.float32), (50, 1000, 8, True, torch.float32),
])
def test_fused_topk_against_oracle(M, E, topk, renorm, dtype):
    g = torch.Generator().manual_seed(M + E)
    logits = torch.randn((M, E), generator=g).to(dtype)
    w_ref, ids_ref = moe_oracle.softmax_topk_ref(logits, topk, renorm)
    hidden = torch.empty((M, 16), device=DEV)
    w, ids = aiter_b200.fused_topk(hidden, logits.to(DEV), topk, renorm)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32
    compare(w, ids, w_ref, ids_ref, f"softmax {M}x{E}")


def test_routing_then_layer_matches_oracle_pipeline():
    """Router -> fused_moe on the device against router -> oracle on the host."""
    from oracle import inputs
    c = inputs.make_config("cfg0", seed=5)
    g = torch.Generator().manual_seed(99)
    logits = torch.randn((c["cfg"]["M"], c["cfg"]["E"]), generator=g)
    w_ref, ids_ref = moe_oracle.softmax_topk_ref(logits, 2, True)
    ref = moe_oracle.fused_moe_ref(c["x"], c["w1_q"], c["w1_scale"], c["w2_q"], c["w2_scale"], w_ref, ids_ref)
    d = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    w, ids = aiter_b200.fused_topk(d["x"], logits.to(DEV), 2, True)
    out = aiter_b200.fused_moe(d["x"], d["w1_q"], d["w2_q"], w, ids, quant_type=aiter_b200.QuantType.per_1x128,
                               w1_scale=d["w1_scale"], w2_scale=d["w2_scale"])
    s = moe_oracle.error_stats(out, ref)
    assert s["frac_within"] >= 0.995 and s["max_abs_excl_one_ulp_over_rms"] <= 0.02, s


def test_routing_errors():
    x = torch.zeros((4, 48), device=DEV)
    w = torch.empty((4, 2), device=DEV)
    ids = torch.empty((4, 2), dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="num_expert_group"):
        aiter_b200.biased_grouped_topk(x, torch.zeros(48, device=DEV), w, ids, 5, 2, True)
    with pytest.raises(RuntimeError, match="fp32 or bf16"):
        aiter_b200.topk_softmax(w, ids, None, x.to(torch.float16), True)
