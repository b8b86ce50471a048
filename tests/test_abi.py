"""The C-ABI library loads on a machine without a GPU and exports what include/*.h declares."""

import ctypes
import glob
import os
import re

import pytest
import torch

from conftest import ROOT

import aiter_b200
from aiter_b200 import _lib, build


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def declared_functions():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names += re.findall(r"\b((?:aiter|b200)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_and_library_agree(lib):
    decl = declared_functions()
    assert len(decl) >= 9
    for name in decl:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert set(_lib.exported_symbols()) == set(decl)


def test_ctypes_signatures_match_header(lib):
    """Every binding passes exactly as many arguments as the header declares."""
    text = ""
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text += re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
    for name, (_res, args) in _lib._SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^)]*)\)", text)
        assert m, name
        params = m.group(1).strip()
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(args), f"{name}: header has {n} parameters, binding passes {len(args)}"


def test_abi_version_and_error_channel(lib):
    assert lib.aiter_ctypes_abi_version() == 4
    lib.aiter_clear_last_error()
    assert lib.aiter_get_last_error() is None
    # a call with a NULL tensor fails with status -1 and a message, without touching a GPU
    st = lib.b200_moe_quant_1x128(None, None, None, None, 1, 0, None)
    assert st == -1
    assert b"input must not be NULL" in lib.aiter_get_last_error()
    lib.aiter_clear_last_error()
    assert lib.aiter_get_last_error() is None


def test_tensor_struct_layout():
    # csrc/include/aiter_tensor.h:8-18 is a 160-byte POD
    assert ctypes.sizeof(_lib.aiter_tensor_t) == 160
    t = torch.zeros((3, 5), dtype=torch.int32)[:, ::2]
    s = _lib.to_aiter(t)
    assert (s.ndim, s.numel_, list(s.shape[:2]), list(s.strides[:2])) == (2, 9, [3, 3], [5, 2])
    assert s.dtype_ == 8 and s.device_id == -1
    assert _lib.to_aiter(None) is None


def test_workspace_size(lib):
    assert aiter_b200.moe_sorting_get_workspace_size(64, 256, 8) == 0
    ws = aiter_b200.moe_sorting_get_workspace_size(8192, 256, 8)
    assert ws == (16 * 256 + 256) * 4


def test_unsupported_options_are_named():
    x = torch.zeros((4, 256), dtype=torch.bfloat16)
    w1 = torch.zeros((2, 512, 256), dtype=torch.float8_e4m3fn)
    w2 = torch.zeros((2, 256, 256), dtype=torch.float8_e4m3fn)
    tw = torch.ones((4, 1))
    ti = torch.zeros((4, 1), dtype=torch.int32)
    QT, AT = aiter_b200.QuantType, aiter_b200.ActivationType
    with pytest.raises(NotImplementedError, match="quant_type"):
        aiter_b200.fused_moe(x, w1, w2, tw, ti, quant_type=QT.per_1x32)
    with pytest.raises(NotImplementedError, match="activation"):
        aiter_b200.fused_moe(x, w1, w2, tw, ti, quant_type=QT.per_1x128, activation=AT.Swiglu)
    with pytest.raises(NotImplementedError, match="bias1"):
        aiter_b200.fused_moe(x, w1, w2, tw, ti, quant_type=QT.per_1x128, bias1=torch.zeros(1))
    with pytest.raises(NotImplementedError, match="splitk"):
        aiter_b200.fused_moe(x, w1, w2, tw, ti, quant_type=QT.per_128x128, splitk=2)
    with pytest.raises(RuntimeError, match="CUDA"):
        aiter_b200.fused_moe(x, w1, w2, tw, ti, quant_type=QT.per_1x128,
                             w1_scale=torch.ones(1), w2_scale=torch.ones(1))
    with pytest.raises(NotImplementedError, match="flat"):
        aiter_b200.moe_sorting(ti, tw, 2, 256, torch.bfloat16, flat=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        aiter_b200.moe_sorting(ti, tw, 2, 256, torch.bfloat16)


def test_enums_match_reference_values():
    QT, AT = aiter_b200.QuantType, aiter_b200.ActivationType
    assert (AT.No, AT.Silu, AT.Gelu, AT.Swiglu, AT.Situv2) == (-1, 0, 1, 2, 3)
    assert [q.value for q in QT] == list(range(8))
    assert QT.per_1x128 == 4 and QT.per_128x128 == 5


def test_registered_operator_fake_and_shuffle_hook():
    """The torch operator propagates shapes on meta tensors (aiter/fused_moe.py:579-619) and
    shuffle_weight keeps the is_shuffled protocol (aiter/ops/shuffle.py:148-209, aiter/fused_moe.py:747)."""
    x = torch.empty((4, 256), dtype=torch.bfloat16, device="meta")
    w1 = torch.empty((2, 512, 256), dtype=torch.float8_e4m3fn, device="meta")
    w2 = torch.empty((2, 256, 256), dtype=torch.float8_e4m3fn, device="meta")
    tw = torch.empty((4, 1), device="meta")
    ti = torch.empty((4, 1), dtype=torch.int32, device="meta")
    out = torch.ops.aiter_b200.fused_moe_(x, w1, w2, tw, ti, None, 0, 4, False, None, None, None, None, None)
    assert out.shape == (4, 256) and out.dtype == torch.bfloat16
    out = torch.ops.aiter_b200.fused_moe_(x.to(torch.float8_e4m3fn), w1, w2, tw, ti, None, 0, 4, False, None, None,
                                          None, None, torch.float16)
    assert out.dtype == torch.float16
    w = torch.zeros((2, 128, 128), dtype=torch.float8_e4m3fn)
    assert aiter_b200.shuffle_weight(w) is w and w.is_shuffled
    with pytest.raises(NotImplementedError):
        aiter_b200.shuffle_weight(w, use_int4=True)
