"""1x128 FP8 quantisation kernel through the C-ABI: bit-exact against pertoken_quant."""

import numpy as np
import pytest
import torch

from conftest import from_bits, load_golden

import aiter_b200
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FP8 = torch.float8_e4m3fn


def test_fixture():
    g = load_golden("quant_1x128.npz")
    x = from_bits(g["x"], torch.bfloat16).to(DEV)
    q, s = aiter_b200.per_group_quant_hip(x, quant_dtype=FP8)
    assert np.array_equal(q.cpu().view(torch.uint8).numpy(), g["q"])
    assert np.array_equal(s.cpu().numpy(), g["scale"])


@pytest.mark.parametrize("rows,cols,std", [(1, 128, 1.0), (7, 7168, 1.0), (513, 2048, 0.05), (64, 4096, 300.0)])
def test_random_bit_exact(rows, cols, std):
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn((rows, cols), generator=g) * std).to(torch.bfloat16)
    x[0, :128] = 0
    q_ref, s_ref = moe_oracle.quant_1x128(x)
    q, s = aiter_b200.get_hip_quant(aiter_b200.QuantType.per_1x128)(x.to(DEV), quant_dtype=FP8)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))


def test_three_dim_input_and_errors():
    x = torch.randn((4, 3, 256), dtype=torch.bfloat16)
    q, s = aiter_b200.per_group_quant_hip(x.to(DEV), quant_dtype=FP8)
    q_ref, s_ref = moe_oracle.quant_1x128(x.view(12, 256))
    assert q.shape == (4, 3, 256) and s.shape == (4, 3, 2)
    assert torch.equal(q.cpu().view(torch.uint8).view(12, 256), q_ref.view(torch.uint8))
    with pytest.raises(RuntimeError, match="multiple of 128"):
        aiter_b200.per_group_quant_hip(torch.zeros((2, 100), dtype=torch.bfloat16, device=DEV), quant_dtype=FP8)


def test_transposed_scales_and_row_limit():
    """transpose_scale (the 1-stage convention, aiter/fused_moe.py:1138-1147) and num_rows/num_rows_factor
    (csrc/kernels/quant_kernels.cu:50-53, 143-146): same codes, scales at [col group * rows + row]; rows past
    num_rows*factor are not written."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn((24, 512), generator=g).to(torch.bfloat16)
    q_ref, s_ref = moe_oracle.quant_1x128(x)
    quant = aiter_b200.get_hip_quant(aiter_b200.QuantType.per_1x128)
    q, s = quant(x.to(DEV), quant_dtype=FP8, transpose_scale=True)
    assert s.shape == (24, 4)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().reshape(-1).view(4, 24).t().contiguous().view(torch.int32), s_ref.view(torch.int32))
    # dynamic row count: 5 * 2 = 10 rows are quantised, the transposed layout uses that row count
    n = torch.tensor([5], dtype=torch.int32, device=DEV)
    sentinel = torch.full((24, 4), -7.0, device=DEV)
    for transposed in (False, True):
        q, s = quant(x.to(DEV), quant_dtype=FP8, transpose_scale=transposed, num_rows=n, num_rows_factor=2)
        assert torch.equal(q[:10].cpu().view(torch.uint8), q_ref[:10].view(torch.uint8))
        got = s.cpu().reshape(-1)[:40]
        want = s_ref[:10].t().contiguous().reshape(-1) if transposed else s_ref[:10].reshape(-1)
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    del sentinel


def test_fp16_input():
    """The reference quantises fp16 activations as well (aiter/fused_moe.py:752-756)."""
    g = torch.Generator().manual_seed(6)
    x = (torch.randn((9, 384), generator=g) * 3).to(torch.float16)
    q_ref, s_ref = moe_oracle.quant_1x128(x)
    q, s = aiter_b200.per_group_quant_hip(x.to(DEV), quant_dtype=FP8)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    qt, st = aiter_b200.per_token_quant_hip(x.to(DEV), quant_dtype=FP8)
    qt_ref, st_ref = moe_oracle.quant_per_token(x)
    assert torch.equal(qt.cpu().view(torch.uint8), qt_ref.view(torch.uint8))
    assert torch.equal(st.cpu().reshape(-1).view(torch.int32), st_ref.reshape(-1).view(torch.int32))
