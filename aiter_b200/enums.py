"""Enums of the fused-MoE API, numerically identical to the reference's
(csrc/include/aiter_enum.h:7-27, exposed as aiter.ActivationType / aiter.QuantType)."""

import enum


class ActivationType(enum.IntEnum):
    No = -1
    Silu = 0
    Gelu = 1
    Swiglu = 2
    Situv2 = 3


class QuantType(enum.IntEnum):
    No = 0
    per_Tensor = 1
    per_Token = 2
    per_1x32 = 3
    per_1x128 = 4
    per_128x128 = 5
    per_256x128 = 6
    per_1024x128 = 7
