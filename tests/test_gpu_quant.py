"""1x128 FP8 quantisation kernel through the C-ABI: bit-exact against pertoken_quant."""

import numpy as np
import pytest
import torch

from conftest import from_bits, load_golden

import aiter_b200
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_fixture():
    g = load_golden("quant_1x128.npz")
    x = from_bits(g["x"], torch.bfloat16).to(DEV)
    q, s = aiter_b200.per_group_quant_hip(x)
    assert np.array_equal(q.cpu().view(torch.uint8).numpy(), g["q"])
    assert np.array_equal(s.cpu().numpy(), g["scale"])


@pytest.mark.parametrize("rows,cols,std", [(1, 128, 1.0), (7, 7168, 1.0), (513, 2048, 0.05), (64, 4096, 300.0)])
def test_random_bit_exact(rows, cols, std):
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn((rows, cols), generator=g) * std).to(torch.bfloat16)
    x[0, :128] = 0
    q_ref, s_ref = moe_oracle.quant_1x128(x)
    q, s = aiter_b200.get_hip_quant(aiter_b200.QuantType.per_1x128)(x.to(DEV))
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))


def test_three_dim_input_and_errors():
    x = torch.randn((4, 3, 256), dtype=torch.bfloat16)
    q, s = aiter_b200.per_group_quant_hip(x.to(DEV))
    q_ref, s_ref = moe_oracle.quant_1x128(x.view(12, 256))
    assert q.shape == (4, 3, 256) and s.shape == (12, 2)
    assert torch.equal(q.cpu().view(torch.uint8).view(12, 256), q_ref.view(torch.uint8))
    with pytest.raises(RuntimeError, match="multiple of 128"):
        aiter_b200.per_group_quant_hip(torch.zeros((2, 100), dtype=torch.bfloat16, device=DEV))
