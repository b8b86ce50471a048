"""Loads the reference's own pure-torch oracle functions from a ROCm/aiter checkout.

TEST INFRASTRUCTURE ONLY, and only usable where a checkout of the reference is present
(``AITER_REFERENCE_ROOT``); it is used by ``tests/golden/make_golden.py`` to pin the
restatement in ``moe_oracle.py`` and to generate the fixtures, never at GPU run time.

``import aiter`` needs ROCm at import time (aiter/jit/utils/cpp_extension.py:138), but the
oracle functions themselves only use torch.  They are cut out of their source files by
``ast`` (no text of the reference is stored here) and executed in a namespace that supplies
the few names they look up: ``dtypes``, ``QuantType``, ``ActivationType``,
``aiter.get_torch_act`` and ``quant_remap``.
"""

from __future__ import annotations

import ast
import enum
import functools
import os
import types

import torch
import torch.nn.functional as F

DEFAULT_ROOT = os.environ.get("AITER_REFERENCE_ROOT", "/root/reference")


class ActivationType(enum.IntEnum):  # csrc/include/aiter_enum.h:7-14
    No = -1
    Silu = 0
    Gelu = 1
    Swiglu = 2
    Situv2 = 3


class QuantType(enum.IntEnum):  # csrc/include/aiter_enum.h:16-26
    No = 0
    per_Tensor = 1
    per_Token = 2
    per_1x32 = 3
    per_1x128 = 4
    per_128x128 = 5
    per_256x128 = 6
    per_1024x128 = 7


def _dtypes_ns():
    # aiter/utility/dtypes.py:11-27 (non-gfx942 mapping: fp8 = e4m3fn)
    ns = types.SimpleNamespace()
    ns.fp32 = torch.float32
    ns.bf16 = torch.bfloat16
    ns.fp16 = torch.float16
    ns.fp8 = torch.float8_e4m3fn
    ns.i8 = torch.int8
    ns.i32 = torch.int32
    ns.i4x2 = getattr(torch, "int4x2", torch.uint8)
    ns.fp4x2 = getattr(torch, "float4_e2m1fn_x2", torch.uint8)
    ns.fp8_e8m0 = getattr(torch, "float8_e8m0fnu", torch.uint8)
    return ns


def _extract(path, names):
    """Compile only the named top-level functions/assignments of ``path``."""
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            keep.append(node)
    found = {n.name for n in keep}
    missing = set(names) - found
    if missing:
        raise RuntimeError(f"{path}: missing {sorted(missing)}")
    return compile(ast.Module(body=keep, type_ignores=[]), path, "exec")


def available(root=DEFAULT_ROOT):
    return os.path.isfile(os.path.join(root, "aiter", "fused_moe.py"))


def load(root=DEFAULT_ROOT):
    """Returns a namespace with the unmodified reference functions:
    torch_moe_stage1, torch_moe_stage2, pertoken_quant, per_tensor_quant, run_torch_moe_sorting,
    biased_grouped_topk_torch."""
    dtypes = _dtypes_ns()
    aiter_ns = types.SimpleNamespace(
        ActivationType=ActivationType, QuantType=QuantType,
        get_torch_act=lambda a: {ActivationType.Silu: F.silu, ActivationType.Gelu: F.gelu}[
            ActivationType(int(a))],
    )
    ns = dict(
        torch=torch, functools=functools, F=F, dtypes=dtypes, aiter=aiter_ns,
        ActivationType=ActivationType, QuantType=QuantType,
        # aiter/fused_moe.py:1310
        quant_remap={QuantType.per_128x128: QuantType.per_1x128},
        BLOCK_SIZE_M=32,
    )
    exec(_extract(os.path.join(root, "aiter", "fused_moe.py"),
                  ["get_inter_dim", "torch_moe_stage1", "torch_moe_stage2", "torch_moe_act"]), ns)
    exec(_extract(os.path.join(root, "aiter", "ops", "quant.py"),
                  ["get_dtype_max", "pertoken_quant", "per_tensor_quant"]), ns)
    exec(_extract(os.path.join(root, "op_tests", "test_moe_sorting.py"),
                  ["run_torch_moe_sorting"]), ns)
    exec(_extract(os.path.join(root, "aiter", "ops", "topk.py"),
                  ["biased_grouped_topk_torch"]), ns)
    aiter_ns.pertoken_quant = ns["pertoken_quant"]
    out = types.SimpleNamespace(**{k: ns[k] for k in (
        "torch_moe_stage1", "torch_moe_stage2", "pertoken_quant", "per_tensor_quant", "run_torch_moe_sorting",
        "biased_grouped_topk_torch")})
    out.QuantType = QuantType
    out.ActivationType = ActivationType
    out.dtypes = dtypes
    return out
