"""The host-side mirror keeps the reference's parameter lists: names, order and defaults of every function a caller
of ROCm/aiter's FP8 fused-MoE path touches are compared with ``tests/golden/reference_signatures.json`` (read from
the reference with ``ast`` by ``tests/golden/make_signatures.py``). CPU only."""

import glob
import inspect
import json
import os
import re

import pytest

import aiter_b200
from aiter_b200 import dtypes
from aiter_b200.enums import ActivationType, QuantType

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIGS = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_signatures.json")))

# what the reference's default expressions evaluate to
_DEFAULT_VALUES = {
    "None": None, "False": False, "True": True, "0": 0, "1": 1, "-1": -1, "1.0": 1.0, "128": 128, "''": "",
    "(16, 16)": (16, 16), "BLOCK_SIZE_M": 32, "ActivationType.Silu": ActivationType.Silu,
    "QuantType.No": QuantType.No, "GateMode.SEPARATED.value": "separated", "dtypes.i8": dtypes.i8,
    "dtypes.fp32": dtypes.fp32,
}

PY_MIRRORS = [k for k in SIGS if not k.startswith("b200_")]


@pytest.mark.parametrize("name", sorted(PY_MIRRORS))
def test_python_mirror_matches_reference(name):
    ref = SIGS[name]["params"]
    sig = inspect.signature(getattr(aiter_b200, name))
    ours = list(sig.parameters.values())
    assert [p.name for p in ours] == [p["name"] for p in ref], f"{name}: {SIGS[name]['reference']}"
    for p, r in zip(ours, ref):
        if r["default"] is None:
            assert p.default is inspect.Parameter.empty, f"{name}.{p.name} must be required"
        else:
            assert r["default"] in _DEFAULT_VALUES, f"add {r['default']!r} to _DEFAULT_VALUES"
            assert p.default == _DEFAULT_VALUES[r["default"]], f"{name}.{p.name}: default {p.default!r} != {r['default']}"


def test_c_sort_entry_binds_argument_for_argument():
    """b200_moe_sorting_fwd takes the arguments of moe_sorting_opus_fwd in the same order (+ the stream)."""
    text = ""
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text += re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
    m = re.search(r"\bb200_moe_sorting_fwd\s*\(([^)]*)\)", text)
    names = [re.split(r"[\s\*]+", p.strip())[-1] for p in m.group(1).split(",")]
    assert names[-1] == "stream"
    assert names[:-1] == [p["name"] for p in SIGS["b200_moe_sorting_fwd"]["params"]]
    m = re.search(r"\bb200_moe_sorting_get_workspace_size\s*\(([^)]*)\)", text)
    names = [re.split(r"[\s\*]+", p.strip())[-1] for p in m.group(1).split(",")]
    assert names == [p["name"] for p in SIGS["moe_sorting_get_workspace_size"]["params"]]


def test_quant_defaults_name_the_unsupported_dtype():
    """The reference defaults quant_dtype to int8, which this library does not build: the error names the argument."""
    import torch
    x = torch.zeros((2, 128), dtype=torch.bfloat16)
    for fn in (aiter_b200.per_group_quant_hip, aiter_b200.per_token_quant_hip, aiter_b200.per_tensor_quant_hip):
        with pytest.raises(NotImplementedError, match="quant_dtype"):
            fn(x)
    with pytest.raises(ValueError, match="static"):
        aiter_b200.per_group_quant_hip(x, scale=torch.ones(1), quant_dtype=dtypes.fp8)
    q = aiter_b200.get_hip_quant(QuantType.per_1x128)
    assert q.func is aiter_b200.per_group_quant_hip and q.keywords == {"group_size": 128}
