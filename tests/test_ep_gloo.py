"""Host logic of the expert-parallel wrapper on two gloo/CPU ranks.

The collectives, the expert mask per rank and the row sharding are the product code
(aiter_b200.ep.ep_fused_moe); the three device steps are replaced by the CPU oracle, which is the
checker here, so the combined result must equal the single-process oracle."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import inputs, moe_oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_quant(x):
    return moe_oracle.quant_1x128(x)


def _oracle_local_layer(a1, a1_scale, w1, w2, topk_weight, topk_ids, expert_mask, w1_scale, w2_scale):
    """fp32 partial sums of this rank's experts (what stage 2 leaves in its accumulator)."""
    M, H = a1.shape
    I = w2.shape[2]
    topk = topk_ids.shape[1]
    ids = moe_oracle.local_expert_ids(topk_ids, expert_mask)
    out1 = moe_oracle.moe_stage1_ref(a1, a1_scale, w1, w1_scale, topk_weight, ids, I)
    a2_q, a2_s = moe_oracle.quant_1x128(out1.view(-1, I))
    return moe_oracle.moe_stage2_ref(a2_q.view(M, topk, I), a2_s.view(M, topk, -1), w2, w2_scale, topk_weight, ids,
                                     dtype=torch.float32)


def _oracle_finalize(acc, dtype):
    return acc.to(dtype)


def _worker(rank, world, port, ret, placed):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from aiter_b200 import ep
        torch.set_num_threads(2)
        c = inputs.make_config("cfg0", seed=0)
        E, M = c["cfg"]["E"], c["cfg"]["M"]
        per, m_local = E // world, M // world
        rows = slice(rank * m_local, (rank + 1) * m_local)
        if placed:
            # an expert -> rank table levelled by the route counts: the rank's weights are its experts in ascending id
            table = ep.balanced_expert_placement(torch.bincount(c["topk_ids"].flatten().long(), minlength=E), world,
                                                 method="lpt")
            sl = ep.local_experts_of(table, rank)
            mask = ep.expert_mask_for_rank(E, rank, world, expert_rank=table)
            assert int(mask.sum()) == per and torch.equal(torch.nonzero(mask).flatten(), sl)
        else:
            table = None
            sl = slice(rank * per, (rank + 1) * per)
            mask = ep.expert_mask_for_rank(E, rank, world)
            assert int(mask.sum()) == per and bool(mask[sl].all())
        out = ep.ep_fused_moe(c["x"][rows], c["w1_q"][sl], c["w2_q"][sl], c["topk_weight"][rows],
                              c["topk_ids"][rows], c["w1_scale"][sl], c["w2_scale"][sl], E,
                              quant=_oracle_quant, local_layer=_oracle_local_layer, finalize=_oracle_finalize,
                              expert_rank=table)
        ret[rank] = out
    finally:
        dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("placed", [False, True])
def test_ep_two_ranks_matches_single_process_oracle(placed):
    world = 2
    port = _free_port()
    manager = mp.Manager()
    ret = manager.dict()
    mp.spawn(_worker, args=(world, port, ret, placed), nprocs=world, join=True)
    c = inputs.make_config("cfg0", seed=0)
    ref = moe_oracle.fused_moe_ref(c["x"], c["w1_q"], c["w1_scale"], c["w2_q"], c["w2_scale"],
                                   c["topk_weight"], c["topk_ids"])
    out = torch.cat([ret[0], ret[1]], dim=0)
    assert out.shape == ref.shape and out.dtype == torch.bfloat16
    s = moe_oracle.error_stats(out, ref)
    # only the fp32 summation order over ranks differs from the single-process sum
    assert s["n_diff"] == s["n_one_ulp"] and s["n_diff"] <= 2e-3 * s["numel"], s


def test_expert_mask_needs_divisible_experts():
    from aiter_b200 import ep
    with pytest.raises(ValueError, match="divisible"):
        ep.expert_mask_for_rank(10, 0, 4)
