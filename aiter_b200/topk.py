"""Router front-ends with the reference's signatures (aiter/ops/topk.py, aiter/fused_moe.py:4058-4129)."""

from __future__ import annotations

import torch

from . import _lib, dtypes


def biased_grouped_topk(gating_output, correction_bias, topk_weights, topk_ids, num_expert_group, topk_group,
                        need_renorm, routed_scaling_factor=1.0):
    """aiter/ops/topk.py:176-215: fills topk_weights [M,topk] fp32 and topk_ids [M,topk] int32 in place."""
    _lib.call("b200_biased_grouped_topk", gating_output.contiguous(), correction_bias.contiguous(), topk_weights,
              topk_ids, int(num_expert_group), int(topk_group), int(bool(need_renorm)), float(routed_scaling_factor),
              device=gating_output.device)
    return topk_weights, topk_ids


def topk_softmax(topk_weights, topk_indices, token_expert_indices, gating_output, need_renorm,
                 num_shared_experts=0, shared_expert_scoring_func=""):
    """aiter/ops/moe_op.py:29-66."""
    if num_shared_experts:
        raise NotImplementedError("topk_softmax: num_shared_experts is not supported")
    _lib.call("b200_topk_softmax", topk_weights, topk_indices, token_expert_indices, gating_output.contiguous(),
              int(bool(need_renorm)), device=gating_output.device)


def fused_topk(hidden_states, gating_output, topk, renormalize, topk_ids=None, topk_weights=None):
    """aiter/fused_moe.py:4058-4129: softmax routing -> (topk_weights fp32, topk_ids int32)."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    M = hidden_states.shape[0]
    dev = hidden_states.device
    if topk_weights is None:
        topk_weights = torch.empty((M, topk), dtype=dtypes.fp32, device=dev)
    if topk_ids is None:
        topk_ids = torch.empty((M, topk), dtype=dtypes.i32, device=dev)
    topk_softmax(topk_weights, topk_ids, None, gating_output, renormalize)
    return topk_weights, topk_ids
