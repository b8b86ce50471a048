"""CPU oracle for the FP8 block-scaled fused-MoE path.

TEST INFRASTRUCTURE ONLY.  Nothing in ``aiter_b200`` (the product) imports this
package; only the test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline
legs of ``bench.py`` do, and only as the checker or the timed CPU baseline.

The functions restate, per expert and in plain torch-on-CPU arithmetic, the
reference's own torch oracle for this path (paths relative to the ROCm/aiter
tree):

* ``aiter/fused_moe.py:3532-3681``  torch_moe_stage1  (block-scale branch)
* ``aiter/fused_moe.py:3684-3811``  torch_moe_stage2  (block-scale branch)
* ``aiter/ops/quant.py:64-94``      pertoken_quant
* ``op_tests/test_moe_2stage.py:184-208``  weight_per_128x128_quant
* ``op_tests/test_moe_sorting.py:45-99``   run_torch_moe_sorting
* ``aiter/ops/topk.py:217-259``     biased_grouped_topk_torch

Parity pin: ``tests/golden/make_golden.py`` runs the unmodified reference
functions (extracted from the reference tree by ``oracle/ref_loader.py``) next to
this restatement on the same seeded inputs, asserts bit-identity, and stores the
reference's outputs as fixtures under ``tests/golden/``.  The CPU test-suite
re-checks the restatement against those fixtures.
"""

from .moe_oracle import (  # noqa: F401
    FP8_MAX,
    quant_1x128,
    quant_weight_128x128,
    quant_per_token,
    moe_sorting_ref,
    moe_stage1_ref,
    moe_stage2_ref,
    fused_moe_ref,
    softmax_topk_ref,
    biased_grouped_topk_ref,
    error_stats,
)
from .inputs import make_config, CONFIGS  # noqa: F401
