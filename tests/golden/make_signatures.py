"""Writes reference_signatures.json: the parameter lists (names, order, defaults as source text) of the reference
functions this package mirrors, read from a checkout of ROCm/aiter with ``ast`` (nothing of it is imported or run).

    AITER_REFERENCE_ROOT=/path/to/aiter python tests/golden/make_signatures.py

The checkout is not available where the tests run, which is why the output is committed;
``tests/test_signatures.py`` compares this package's functions with it.
"""

from __future__ import annotations

import ast
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

# (file in the reference tree, function) -> name of the mirror in aiter_b200
TARGETS = [
    ("aiter/fused_moe.py", "fused_moe", "fused_moe"),
    ("aiter/fused_moe.py", "moe_sorting", "moe_sorting"),
    ("aiter/fused_moe.py", "fused_topk", "fused_topk"),
    ("aiter/ops/quant.py", "per_group_quant_hip", "per_group_quant_hip"),
    ("aiter/ops/quant.py", "per_token_quant_hip", "per_token_quant_hip"),
    ("aiter/ops/quant.py", "per_tensor_quant_hip", "per_tensor_quant_hip"),
    ("aiter/ops/moe_sorting_opus.py", "moe_sorting_opus_get_workspace_size", "moe_sorting_get_workspace_size"),
    ("aiter/ops/moe_sorting_opus.py", "moe_sorting_opus_fwd", "b200_moe_sorting_fwd"),
    ("aiter/ops/topk.py", "biased_grouped_topk", "biased_grouped_topk"),
    ("aiter/ops/moe_op.py", "topk_softmax", "topk_softmax"),
    ("aiter/ops/shuffle.py", "shuffle_weight", "shuffle_weight"),
]


def params_of(path, func):
    tree = ast.parse(open(path).read())
    nodes = [n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef) and n.name == func]
    assert nodes, f"{func} not found in {path}"
    node = nodes[0]
    a = node.args
    assert not a.posonlyargs and not a.kwonlyargs and a.vararg is None and a.kwarg is None, (path, func)
    defaults = [None] * (len(a.args) - len(a.defaults)) + [ast.unparse(d) for d in a.defaults]
    return [{"name": arg.arg, "default": d} for arg, d in zip(a.args, defaults)], node.lineno


def main():
    root = os.environ.get("AITER_REFERENCE_ROOT")
    if not root:
        sys.exit("set AITER_REFERENCE_ROOT to a checkout of ROCm/aiter")
    out = {}
    for rel, func, mirror in TARGETS:
        params, line = params_of(os.path.join(root, rel), func)
        out[mirror] = {"reference": f"{rel}:{line}", "function": func, "params": params}
    with open(os.path.join(HERE, "reference_signatures.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"wrote {len(out)} signatures")


if __name__ == "__main__":
    main()
