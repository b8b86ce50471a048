"""aiter_b200: the FP8 block-scaled fused-MoE path of ROCm/aiter, rebuilt for NVIDIA B200.

Public surface (same names as the reference's): ``fused_moe``, ``moe_sorting``, ``QuantType``,
``ActivationType``, ``dtypes``, ``get_hip_quant`` / ``per_group_quant_hip``.
"""

from . import dtypes  # noqa: F401
from .enums import ActivationType, QuantType  # noqa: F401
from .fused_moe import (  # noqa: F401
    check_device_status,
    fused_moe,
    fused_moe_,
    shuffle_weight,
    get_hip_quant,
    moe_sorting,
    moe_sorting_get_workspace_size,
    per_group_quant_hip,
    per_tensor_quant_hip,
    per_token_quant_hip,
)

from .topk import biased_grouped_topk, fused_topk, topk_softmax  # noqa: F401,E402

__all__ = [
    "biased_grouped_topk", "fused_topk", "topk_softmax",
    "ActivationType", "QuantType", "dtypes", "fused_moe", "fused_moe_", "shuffle_weight", "moe_sorting",
    "moe_sorting_get_workspace_size", "get_hip_quant", "per_group_quant_hip", "per_token_quant_hip", "per_tensor_quant_hip", "check_device_status",
]
