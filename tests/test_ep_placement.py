"""Expert -> rank placement from routing statistics (host logic, no GPU)."""

import pytest
import torch

from aiter_b200 import ep
from oracle import inputs


def _group_limited_counts(M=4096, E=64, topk=8, seed=11):
    _tw, ti = inputs.make_routing("dsv3", M, E, topk, seed)
    return ti, torch.bincount(ti.flatten().long(), minlength=E)


@pytest.mark.parametrize("method", ["swap", "lpt"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_placement_levels_the_ranks(method, world):
    ti, counts = _group_limited_counts()
    E = counts.numel()
    table = ep.balanced_expert_placement(counts, world, method=method)
    assert table.dtype == torch.int32 and table.shape == (E,)
    assert torch.equal(torch.bincount(table.long(), minlength=world), torch.full((world,), E // world))
    load = torch.zeros(world, dtype=torch.long).index_add_(0, table.long(), counts)
    contiguous = counts.view(world, E // world).sum(1)
    assert load.max() <= contiguous.max()
    assert load.max() <= 1.05 * load.sum() / world
    # the rank's experts, ascending, are what local_experts_of lists
    for r in range(world):
        mine = ep.local_experts_of(table, r)
        assert torch.equal(mine, torch.nonzero(table == r).flatten()) and mine.numel() == E // world


def test_swap_moves_few_experts_and_keeps_tokens_on_few_ranks():
    ti, counts = _group_limited_counts()
    E, world = counts.numel(), 8
    home = torch.arange(E, dtype=torch.int32) // (E // world)
    swap = ep.balanced_expert_placement(counts, world, method="swap")
    lpt = ep.balanced_expert_placement(counts, world, method="lpt")
    moved = lambda t: int((t != home).sum())
    ranks_per_token = lambda t: float(torch.zeros((ti.shape[0], world), dtype=torch.bool)
                                      .scatter_(1, t[ti.long()].long(), True).sum(1).float().mean())
    assert moved(swap) < moved(lpt)
    assert ranks_per_token(home) <= ranks_per_token(swap) <= ranks_per_token(lpt)


def test_level_counts_are_left_alone_and_bad_arguments_raise():
    counts = torch.full((16,), 100)
    assert torch.equal(ep.balanced_expert_placement(counts, 4, method="swap"), torch.arange(16, dtype=torch.int32) // 4)
    with pytest.raises(ValueError):
        ep.balanced_expert_placement(torch.ones(10), 4)
    with pytest.raises(ValueError):
        ep.balanced_expert_placement(torch.ones(16), 4, method="random")
