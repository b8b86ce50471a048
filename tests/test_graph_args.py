"""CapturedLayer argument checks that need no GPU."""

import pytest
import torch

from aiter_b200.graph import CapturedLayer


def test_inputs_must_be_cuda_tensors():
    with pytest.raises(ValueError):
        CapturedLayer(lambda x: x, torch.zeros(4))
    with pytest.raises(ValueError):
        CapturedLayer(lambda: torch.zeros(1))
    with pytest.raises(ValueError):
        CapturedLayer(lambda x: x, 3)
