"""The benchmark draws its own synthetic inputs (its GPU arm imports nothing from oracle/): they must be the
format the oracle and the parity tests use."""

import importlib.util
import os

import torch

from oracle import inputs, moe_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_weight_quantisation_matches_the_oracle_format():
    b = _bench()
    q, s = b.quantise_weights(3, 256, 384, 7, "cpu")
    q_ref, s_ref = inputs.make_weights(3, 256, 384, 7)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s, s_ref)


def test_host_routing_is_the_oracle_router_on_the_bench_logits():
    b = _bench()
    x, tw, ti = b.make_tokens(64, seed=1)
    _x, logits, bias = b.router_inputs(64, seed=1)
    tw_ref, ti_ref = moe_oracle.biased_grouped_topk_ref(logits, bias, b.TOPK, True, 8, 4, routed_scaling_factor=2.5)
    assert torch.equal(ti, ti_ref) and torch.equal(tw, tw_ref)
    assert x.shape == (64, b.H) and x.dtype == torch.bfloat16
    # a token's experts lie in at most 4 of the 8 groups
    groups = (ti // (b.E // 8)).tolist()
    assert max(len(set(g)) for g in groups) <= 4
