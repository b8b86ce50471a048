"""The bounded device-side waits of the GEMM kernels, exercised without faulting or hanging anything.

``b200_moe_debug_config`` stalls the weight-loading role of the next launches and shortens the wait limit to about a
millisecond: nothing is ever in flight, every waiting role runs out of time on its own clock, each CTA winds down, frees
its tensor memory and sets the status word; ``check_device_status`` raises. The context stays usable: with the settings
restored, the same call gives bit-for-bit what it gave before."""

import pytest
import torch

import aiter_b200
from aiter_b200 import _lib
from oracle import inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layer(c):
    # doweight in stage 2 only, one row block per expert: a single GEMM tile order, so two runs agree bit for bit
    return aiter_b200.fused_moe(c["x"], c["w1_q"], c["w2_q"], c["topk_weight"], c["topk_ids"],
                                quant_type=aiter_b200.QuantType.per_1x128, w1_scale=c["w1_scale"], w2_scale=c["w2_scale"])


def test_waits_run_out_and_the_next_call_is_unchanged():
    c = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in inputs.make_config("cfg0", seed=0).items()}
    c["topk_ids"] = c["topk_ids"][:, :1].contiguous()      # one route per token: no fp32 reduction order to vary
    c["topk_weight"] = c["topk_weight"][:, :1].contiguous()
    before = _layer(c)
    torch.cuda.synchronize()
    aiter_b200.check_device_status()
    try:
        _lib.call_plain("b200_moe_debug_config", 2_000_000, 1)    # ~1 ms at 1.9 GHz, producer stalled
        _layer(c)
        torch.cuda.synchronize()                                   # the kernels end by themselves
        with pytest.raises(RuntimeError, match="gave up on a device-side wait"):
            aiter_b200.check_device_status()
    finally:
        _lib.call_plain("b200_moe_debug_config", 0, 0)
    aiter_b200.check_device_status()                               # the word was cleared by the raise
    after = _layer(c)
    torch.cuda.synchronize()
    aiter_b200.check_device_status()
    assert torch.equal(before.view(torch.int16), after.view(torch.int16))
    assert float(after.float().abs().max()) > 0
