"""The allocation-free sort entry point against the regular one, through the C-ABI.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test. Works in a fresh process and after the other GPU tests alike."""

import pytest
import torch

import aiter_b200
from aiter_b200 import _lib
from oracle import inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def sort_outputs(M, topk, E, unit):
    P = M * topk + E * unit - topk
    return (torch.empty(P, dtype=torch.int32, device=DEV), torch.empty(P, dtype=torch.float32, device=DEV),
            torch.empty((P + unit - 1) // unit, dtype=torch.int32, device=DEV),
            torch.empty(2, dtype=torch.int32, device=DEV))


def run_both(M, E, topk, unit, kind, seed, mask=None):
    w, ids = inputs.make_routing(kind, M, E, topk, seed)
    w, ids = w.to(DEV), ids.to(DEV)
    ref = aiter_b200.moe_sorting(ids, w, E, 64, torch.bfloat16, unit, mask, accumulate=False)
    out = sort_outputs(M, topk, E, unit)
    # poison the outputs so a kernel that wrote nothing cannot pass
    for t in out:
        t.fill_(-7)
    _lib.call("b200_moe_sorting_fwd_noalloc", ids, w, out[0], out[1], out[2], out[3], None, E, unit, mask, None,
              None, device=torch.device(DEV))
    torch.cuda.synchronize()
    for name, a, b in zip(("sorted_ids", "sorted_weights", "sorted_expert_ids", "num_valid_ids"), out, ref[:4]):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32)), name


def test_no_alloc_sort_matches_regular_sort_twice():
    # two calls in a row share the built-in scratch: the second (other size, other routing, a mask)
    # must not see anything of the first
    run_both(8192, 256, 8, 128, "dsv3", seed=0)
    mask = (torch.arange(128, device=DEV) % 3 != 0).to(torch.int32)
    run_both(5000, 128, 8, 64, "zipf", seed=1, mask=mask)
    # the single-CTA path needs no scratch at all and goes through the same entry point
    run_both(64, 256, 8, 128, "dsv3", seed=2)


def test_no_alloc_sort_rejects_oversized_problems():
    M, topk, E, unit = 40000, 8, 64, 32   # 320000 routes > 262144
    ids = torch.zeros((M, topk), dtype=torch.int32, device=DEV)
    w = torch.ones((M, topk), device=DEV)
    out = sort_outputs(M, topk, E, unit)
    with pytest.raises(RuntimeError, match="too large for the built-in scratch"):
        _lib.call("b200_moe_sorting_fwd_noalloc", ids, w, out[0], out[1], out[2], out[3], None, E, unit, None, None,
                  None, device=torch.device(DEV))
