"""moe_sorting through the C-ABI against the oracle and the reference-made fixtures: bit-exact."""

import numpy as np
import pytest
import torch

from conftest import bits_equal, load_golden
from test_oracle_golden import sorting_sweep_cases

import aiter_b200
from oracle import inputs, moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_sort(ids, w, E, B, mask=None, nl=None, **kw):
    d = lambda t: None if t is None else t.to(DEV)
    return aiter_b200.moe_sorting(d(ids), d(w), E, 256, torch.bfloat16, B, d(mask), d(nl), **kw)


def check(out, exp, tag=""):
    names = ("sorted_ids", "sorted_weights", "sorted_expert_ids", "num_valid_ids")
    for name, a, b in zip(names, out, exp):
        assert bits_equal(a, b), f"{tag}: {name} differs"


def test_known_answers():
    g = load_golden("sorting_kat.npz")
    ids, w, mask = (torch.from_numpy(g[k]) for k in ("topk_ids", "topk_weights", "mask"))
    for tag, m in (("plain", None), ("masked", mask)):
        out = run_sort(ids, w, 6, 4, m)
        exp = tuple(torch.from_numpy(g[f"{tag}_{k}"]) for k in
                    ("sorted_ids", "sorted_weights", "sorted_expert_ids", "num_valid"))
        check(out, exp, tag)
    # op_tests/test_moe_local_expert_ids.py:13-63
    ids3, mask3 = torch.from_numpy(g["ids3"]), torch.from_numpy(g["mask3"])
    w3 = torch.ones(ids3.shape)
    *_, local = run_sort(ids3, w3, 6, 8, mask3, return_local_topk_ids=True)
    assert local.cpu().tolist() == [[-1, 0, -1], [1, 2, -1], [-1, -1, 1]]
    *_, local = run_sort(ids3, w3, 6, 8, None, return_local_topk_ids=True)
    assert torch.equal(local.cpu(), ids3)


def test_fixture_sweep():
    n = 0
    for k, (ids, w, E, B, mask, nl), exp in sorting_sweep_cases():
        check(run_sort(ids, w, E, B, mask, nl), exp, k)
        n += 1
    assert n == 21


@pytest.mark.parametrize("M,E,topk,B", [
    (1, 8, 2, 128), (3, 256, 8, 128), (31, 40, 6, 32), (2049, 256, 8, 128),   # single-CTA path
    (2050, 256, 8, 128), (8192, 256, 8, 128), (16384, 128, 8, 128), (5000, 385, 7, 64),
    (3000, 1024, 8, 16),                                                      # multi-CTA path
])
def test_random_against_oracle(M, E, topk, B):
    g = torch.Generator().manual_seed(M * 131 + E)
    sc = torch.rand((M, E), generator=g)
    w, ids = torch.topk(sc, topk, dim=-1)
    ids = ids.to(torch.int32)
    mask = (torch.rand(E, generator=g) > 0.3).to(torch.int32)
    nl = torch.tensor([max(1, (M * 2) // 3)], dtype=torch.int32)
    for tag, m, n in (("plain", None, None), ("mask", mask, None), ("local", None, nl), ("both", mask, nl)):
        exp = moe_oracle.moe_sorting_ref(ids, w, E, B, m, n)
        check(run_sort(ids, w, E, B, m, n), exp, f"{M}x{E}x{topk}/{B} {tag}")


def test_no_tokens():
    """M = 0: every slot of the padded output is a pad, no block is valid."""
    ids, w = torch.zeros((0, 2), dtype=torch.int32), torch.zeros((0, 2), dtype=torch.float32)
    exp = moe_oracle.moe_sorting_ref(ids, w, 8, 128)
    check(run_sort(ids, w, 8, 128), exp, "no tokens")


def test_skewed_routing_and_empty_experts():
    w, ids = inputs.make_routing("zipf", 4096, 128, 8, seed=5)
    exp = moe_oracle.moe_sorting_ref(ids, w, 128, 128)
    check(run_sort(ids, w, 128, 128), exp, "zipf")
    # every route to one expert; all other experts empty
    ids = torch.zeros((700, 1), dtype=torch.int32) + 3
    w = torch.rand((700, 1))
    exp = moe_oracle.moe_sorting_ref(ids, w, 16, 128)
    check(run_sort(ids, w, 16, 128), exp, "one expert")


def test_moe_buf_is_zeroed_and_placeholder():
    w, ids = inputs.make_routing("softmax", 300, 8, 2, seed=1)
    ids, w = ids.to(DEV), w.to(DEV)
    torch.full((300 * 1000,), 7.0, device=DEV)  # dirty the allocator's pool
    *_, buf = aiter_b200.moe_sorting(ids, w, 8, 1000, torch.bfloat16, 32)
    assert buf.shape == (300, 1000) and buf.dtype == torch.bfloat16
    assert int((buf.view(torch.int16) != 0).sum()) == 0
    *_, buf = aiter_b200.moe_sorting(ids, w, 8, 1000, torch.bfloat16, 32, accumulate=False)
    assert buf.shape == (0, 0)
    # multi-CTA path with a buffer whose byte size is not a multiple of 16
    w, ids = inputs.make_routing("softmax", 9001, 8, 2, seed=2)
    *_, buf = aiter_b200.moe_sorting(ids.to(DEV), w.to(DEV), 8, 3, torch.float16, 32)
    assert buf.shape == (9001, 3) and int((buf.view(torch.int16) != 0).sum()) == 0
    # the fp32 accumulator of the layer: cleared beside the scan kernel, whatever the pool held before
    del buf
    dirty = torch.full((9001 * 512,), float("nan"), device=DEV)
    del dirty
    *_, buf = aiter_b200.moe_sorting(ids.to(DEV), w.to(DEV), 8, 512, torch.float32, 128)
    assert buf.shape == (9001, 512) and buf.dtype == torch.float32
    assert int((buf.view(torch.int32) != 0).sum()) == 0


def test_errors_are_reported_not_crashed():
    ids = torch.zeros((4, 2), dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="topk_weights must be FP32"):
        aiter_b200.moe_sorting(ids, torch.ones((4, 2), dtype=torch.float16, device=DEV), 8, 64, torch.bfloat16)
    with pytest.raises(RuntimeError, match="num_experts"):
        aiter_b200.moe_sorting(ids, torch.ones((4, 2), device=DEV), 5000, 64, torch.bfloat16)
