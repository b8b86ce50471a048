"""dtype aliases of the reference (aiter/utility/dtypes.py:11-27); fp8 is OCP e4m3fn as on
every non-gfx942 target."""

import torch

fp32 = torch.float32
fp16 = torch.float16
bf16 = torch.bfloat16
fp8 = torch.float8_e4m3fn
i8 = torch.int8
u8 = torch.uint8
i16 = torch.int16
i32 = torch.int32
u32 = torch.uint32
i64 = torch.int64

# AiterDtype codes (csrc/include/aiter_enum.h:36-52)
AITER_DTYPE = {
    torch.float8_e4m3fn: 0,
    torch.float16: 2,
    torch.bfloat16: 3,
    torch.float32: 4,
    torch.uint32: 7,
    torch.int32: 8,
    torch.int16: 9,
    torch.int8: 10,
    torch.uint8: 11,
    torch.int64: 12,
    torch.uint64: 13,
}
