#!/usr/bin/env python
"""Benchmark of the FP8 block-scaled fused-MoE layer (DeepSeek-V3 shape) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the layer over one batch of synthetic tokens (seeded N(0,1) activations,
N(0,1/sqrt(K)) weights quantised to e4m3 per 128x128 block, DeepSeek-V3 grouped top-8 routing).
Headline workload: M=8192 tokens, H=7168, I=2048, E=256, topk=8 (prefill); the M=64 decode case is
measured in the same run and reported under "decode".  With N GPUs the experts are sharded
(expert parallelism: token dispatch, local layer, combine of the fp32 partial sums; over peer memory or
NCCL) and the total work stays fixed, so scaling is "strong".  Rank 0 prints ONE JSON line.

Beside the headline the same run measures, through the same public calls: the M=64 decode layer ("decode", at
every N), the Mixtral-shaped per_Token layer and the Qwen3-shaped skewed-routing sweep ("other_configs"), and for
N > 1 checks a handful of rank-0 output rows against the CPU oracle ("parity_check", outside every timed region).

`--impl reference` times the CPU oracle (the reference's torch arithmetic restated per expert) on
the host cores over a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, I, E, TOPK = 7168, 2048, 256, 8
M_PREFILL, M_DECODE = 8192, 64
WORKLOAD = "dsv3_fp8_blockscale_moe_prefill_M8192_H7168_I2048_E256_topk8"
METRIC = "DSV3 FP8-blockscale fused_moe TFLOP/s (M=8192)"


# DRAM traffic of one stage-1 launch (dram__bytes_read.sum + dram__bytes_write.sum), per expert, from an `ncu --set
# full` capture of a small case with the headline's routes per expert; a full launch is this times the expert count
# (the weights, which make up the traffic, grow with it). Refresh when the GEMM kernel or its tile walk changes.
STAGE1_DRAM_BYTES_PER_EXPERT = 1.172e9 / 32
STAGE1_DRAM_CAPTURE = "ncu --set full, moe_gemm_kernel<1>, M=1024 E=32 H=7168 I=2048 topk=8 (256 routes per expert), 2026-11-25"


def flops(M):
    return 6.0 * M * TOPK * H * I


def algorithmic_bytes(M, n_active):
    per_expert = 3 * H * I + 3 * H * I // 16384 * 4
    return n_active * per_expert + 4 * M * H + 8 * M * TOPK


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def _nvml_handle(pynvml, cuda_index):
    """NVML handle of CUDA device ``cuda_index`` (by PCI bus id: the two index spaces differ under CUDA_VISIBLE_DEVICES)."""
    pr = torch.cuda.get_device_properties(cuda_index)
    bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
    try:
        return pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
    except TypeError:
        return pynvml.nvmlDeviceGetHandleByPciBusId(bus)


def bind_near_gpu(cuda_index):
    """Restricts this process to the host cores NVML reports as local to the GPU (its NUMA node), so that the pinned
    step buffers are allocated on that node and the copy threads run there. Reads NVML only; changes nothing but this
    process's own CPU affinity. Returns a short description for the bench line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = _nvml_handle(pynvml, cuda_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        want = near & allowed
        if not want or want == allowed:
            return f"unchanged ({len(allowed)} cores allowed, {len(near)} local to the GPU)"
        os.sched_setaffinity(0, want)
        return f"{len(want)} of {len(allowed)} allowed cores, those local to the GPU"
    except Exception as e:   # noqa: BLE001 - a placement hint: never a reason to fail the bench
        return f"unchanged ({type(e).__name__}: {e})"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        # NVML in a thread of this process (what nvidia-smi itself reads): a sample every few milliseconds, so that
        # even a timed region of some tens of milliseconds (8 ranks) is covered; nvidia-smi -lms as the fallback
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = _nvml_handle(pynvml, self.gpu)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.stop_flag = False
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:   # noqa: BLE001 - any NVML problem: use the command-line tool
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(reasons_fn(self.handle))
                self.rows.append([mhz, [n for n, b in bits.items() if mask & b]])
            except Exception:   # noqa: BLE001
                pass
            time.sleep(0.004)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.t.join(timeout=2)
            sm = [r[0] for r in self.rows]
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            reasons = [n for n in names if any(n in r[1] for r in self.rows)]
            return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=self.max_mhz, reasons=reasons,
                        samples=len(sm), source="NVML, one sample per 4 ms")
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm), source="nvidia-smi -lms 100")


# ------------------------------------------------------------------------------------------ inputs
def quantise_weights(E_, N, K, seed, device):
    """[E_, N, K] ~ N(0, 1/sqrt(K)) drawn on `device` one expert at a time and quantised to e4m3 per 128x128 block
    with scale = amax/448 (0 -> 1): the weight format of the reference's tests (op_tests/test_moe_2stage.py:184-208)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    q = torch.empty((E_, N, K), dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty((E_, N // 128, K // 128), dtype=torch.float32, device=device)
    std = 1.0 / (K ** 0.5)
    for e in range(E_):
        w = torch.randn((N, K), generator=g, dtype=torch.float32, device=device) * std
        blocks = w.view(N // 128, 128, K // 128, 128)
        amax = blocks.abs().amax(dim=(1, 3), keepdim=True)
        scale = amax / 448.0
        scale[scale == 0] = 1.0
        q[e] = (blocks / scale).view(N, K).to(torch.float8_e4m3fn)
        s[e] = scale.view(N // 128, K // 128)
    return q, s


def make_layer(device, rank, world, seed=0):
    """This rank's expert slice (weights drawn and quantised on the device)."""
    e_local = E // world
    w1_q, w1_s = quantise_weights(e_local, 2 * I, H, seed + 1 + 1000 * rank, device)
    w2_q, w2_s = quantise_weights(e_local, H, I, seed + 2 + 1000 * rank, device)
    return w1_q, w1_s, w2_q, w2_s


def router_inputs(M, seed=0, bias=None):
    """Seeded activations, router logits ~ N(0,1) and correction bias ~ N(0, 0.1) (host generator). ``bias``: reuse
    the correction bias of another batch (it is a model parameter: a calibration batch for the expert placement has
    the model's bias, not one of its own)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, H), generator=g, dtype=torch.float32).to(torch.bfloat16)
    g = torch.Generator().manual_seed(seed + 3)
    logits = torch.randn((M, E), generator=g, dtype=torch.float32)
    own_bias = torch.randn((E,), generator=g, dtype=torch.float32) * 0.1
    return x, logits, own_bias if bias is None else bias


def make_tokens(M, seed=0, device=None, bias=None):
    """x [M,H] bf16 and DeepSeek-V3 routing (8 groups, top-4 groups, top-8 experts, renormalised, x2.5): computed by
    this library's own router kernel on `device`; on the host (the CPU legs, device=None) by the oracle's router."""
    x, logits, bias = router_inputs(M, seed, bias)
    if device is None:
        from oracle import moe_oracle
        tw, ti = moe_oracle.biased_grouped_topk_ref(logits, bias, TOPK, True, 8, 4, routed_scaling_factor=2.5)
        return x, tw, ti
    import aiter_b200
    tw = torch.empty((M, TOPK), dtype=torch.float32, device=device)
    ti = torch.empty((M, TOPK), dtype=torch.int32, device=device)
    aiter_b200.biased_grouped_topk(logits.to(device), bias.to(device), tw, ti, 8, 4, True, 2.5)
    return x, tw.cpu(), ti.cpu()


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_sample_step(x, tw, ti, w1_q, w1_s, w2_q, w2_s, n_exp):
    """Oracle on the routes of the first ``n_exp`` experts (all tokens, 1/(E/n_exp) of the layer)."""
    from oracle import moe_oracle
    mask = torch.zeros(E, dtype=torch.int32)
    mask[:n_exp] = 1
    t0 = time.perf_counter()
    moe_oracle.fused_moe_ref(x, w1_q[:n_exp], w1_s[:n_exp], w2_q[:n_exp], w2_s[:n_exp], tw, ti, expert_mask=mask)
    dt = time.perf_counter() - t0
    routes = int((ti < n_exp).sum())
    return dt, 6.0 * routes * H * I


def cpu_baseline(n_exp=8, steps=1, warmup=0, seed=0):
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    x, tw, ti = make_tokens(M_PREFILL, seed)
    w1_q, w1_s = quantise_weights(n_exp, 2 * I, H, seed + 1, "cpu")
    w2_q, w2_s = quantise_weights(n_exp, H, I, seed + 2, "cpu")
    times, fl = [], 0.0
    for i in range(warmup + steps):
        dt, fl = cpu_sample_step(x, tw, ti, w1_q, w1_s, w2_q, w2_s, n_exp)
        if i >= warmup:
            times.append(dt)
    t = sum(times) / len(times)
    return dict(value=fl / t / 1e12, unit="TFLOP/s", cores=cores, kind="port",
                sample=f"routes of experts 0..{n_exp - 1} of {E} over all {M_PREFILL} tokens "
                       f"({fl / flops(M_PREFILL):.4f} of the layer's FLOPs), {len(times)} run(s), {t:.2f} s each",
                seconds_per_step=t)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_exp = 32
    # each step is a bounded sample (1/8 of the experts, all tokens); at most ~2 minutes of steps
    probe = cpu_baseline(n_exp=n_exp, steps=1, warmup=0)
    steps = max(1, min(args.steps, int(120.0 / max(probe["seconds_per_step"], 1e-3))))
    cb = cpu_baseline(n_exp=n_exp, steps=steps, warmup=0) if steps > 1 else probe
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (e4m3 codes dequantised)",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": cb["sample"]},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "steps_run": steps,
    }
    emit(line)


# ------------------------------------------------------------------------------------------ GPU arm
def timed(fn, steps, warmup, sync, profile=False):
    for _ in range(warmup):
        fn()
    sync()
    if profile:
        torch.cuda.profiler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        fn()
        ev[i + 1].record()
    sync()
    if profile:
        torch.cuda.profiler.stop()
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]


def timed_e2e_pipelined(layer, host_in, host_out2, dev, steps, warmup, sync, static_out=False):
    """End-to-end steps as a serving loop runs them: every step copies its inputs from pinned host
    memory and its result back to pinned host memory; the copies of neighbouring steps overlap the
    compute on two copy streams (double-buffered device inputs, double-buffered host outputs).
    Returns the total time of `steps` steps in ms (CUDA events on the compute stream, which waits
    for the last device-to-host copy before the end event).
    ``static_out``: the layer returns the same tensor every step (a replayed graph's output); it is copied into
    one of two preallocated device buffers before the next replay overwrites it, so the loop allocates nothing."""
    comp = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dbuf = [[torch.empty_like(t, device=dev) for t in host_in] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    obuf = [torch.empty(host_out2[0].shape, dtype=host_out2[0].dtype, device=dev) for _ in range(2)] if static_out else None
    for ev in out_done:
        ev.record(s_out)

    def run(n):
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(comp_done[b])          # the step that last read this input buffer
                for d, h in zip(dbuf[b], host_in):
                    d.copy_(h, non_blocking=True)
                in_ready[b].record(s_in)
            comp.wait_event(in_ready[b])
            out = layer(*dbuf[b])
            if static_out:
                comp.wait_event(out_done[b])           # the device-to-host copy that last read this buffer
                obuf[b].copy_(out, non_blocking=True)
                out = obuf[b]
            comp_done[b].record(comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                host_out2[b].copy_(out, non_blocking=True)
                if not static_out:
                    out.record_stream(s_out)
                out_done[b].record(s_out)

    for ev in comp_done:
        ev.record(comp)
    run(warmup)
    comp.wait_stream(s_out)
    sync()
    for ev in comp_done:
        ev.record(comp)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(comp)
    run(steps)
    comp.wait_stream(s_out)
    e1.record(comp)
    sync()
    return e0.elapsed_time(e1)


def kernel_breakdown(fm, dev_args, reps=5):
    """Average device time of each kernel of the layer, from CUDA events on the launch stream."""
    acc = {}
    for _ in range(reps):
        timers = []
        fm.fused_moe_stages(*dev_args, timers=timers)
        torch.cuda.synchronize()
        for (n0, e0), (_n1, e1) in zip(timers[:-1], timers[1:]):
            acc.setdefault(n0, []).append(e0.elapsed_time(e1))
    return {k: sum(v) / len(v) for k, v in acc.items()}


def library_fp8_gemm_tflops(dev, n=8192, iters=20):
    """Throughput of the vendor library's dense e4m3 GEMM (n^3, tensor-wise scales, bf16 out), event-timed here:
    the FP8 tensor-core rate a library kernel reaches on this GPU in this run, reported beside the roofline
    denominator. None if the call is unavailable."""
    try:
        a = torch.randn((n, n), device=dev).to(torch.float8_e4m3fn)
        b = torch.randn((n, n), device=dev).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev, dtype=torch.float32)

        def f():
            return torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        for _ in range(5):
            f()
        torch.cuda.synchronize(dev)
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (statistics.median(ts) * 1e-3) / 1e12
    except Exception:   # noqa: BLE001 - a missing or changed private API must not break the bench
        return None


# ------------------------------------------------------------------------------------------ other configurations
def quantise_weights_per_channel(E_, N, K, seed, device):
    """[E_, N, K] ~ N(0, 1/sqrt(K)) quantised to e4m3 with one scale per output channel (QuantType.per_Token weights,
    op_tests/test_moe_2stage.py:213-214)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    q = torch.empty((E_, N, K), dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty((E_, N, 1), dtype=torch.float32, device=device)
    std = 1.0 / (K ** 0.5)
    for e in range(E_):
        w = torch.randn((N, K), generator=g, dtype=torch.float32, device=device) * std
        scale = w.abs().amax(dim=1, keepdim=True) / 448.0
        scale[scale == 0] = 1.0
        q[e] = (w / scale).to(torch.float8_e4m3fn)
        s[e] = scale
    return q, s


def zipf_routing(M, E_, topk, seed):
    """topk distinct experts per token from Zipf(s=1.2) over a seeded permutation of the expert ids, weights =
    softmax of N(0,1) over the chosen experts (BASELINE.json's skewed-routing sweep)."""
    g = torch.Generator().manual_seed(seed + 3)
    perm = torch.randperm(E_, generator=g)
    p = 1.0 / torch.arange(1, E_ + 1, dtype=torch.float64) ** 1.2
    p = (p / p.sum()).to(torch.float32)
    ranks = torch.multinomial(p.expand(M, E_), topk, replacement=False, generator=g)
    ids = perm[ranks].to(torch.int32)
    w = torch.softmax(torch.randn((M, topk), generator=g, dtype=torch.float32), dim=-1)
    return w, ids


def median_ms(fn, sync, steps=10, warmup=3):
    return statistics.median(timed(fn, steps, warmup, sync))


def bench_other_configs(dev, rank, world, sync, max_over_ranks, exchange, steps):
    """Config 3 (Mixtral-8x7B shape, QuantType.per_Token, M=4096) and config 4 (Qwen3-235B-A22B shape, Zipf(1.2) routing,
    M in {1, 16, 128, 1024, 16384}) through the same public calls; N > 1: expert parallel over the N ranks."""
    import aiter_b200
    from aiter_b200 import ep
    QT = aiter_b200.QuantType
    out = {}
    # ---- config 3
    Hm, Im, Em, Km, Mm = 4096, 14336, 8, 2, 4096
    if Em % world == 0 and Mm % world == 0:
        el = Em // world
        w1_q, w1_s = quantise_weights_per_channel(el, 2 * Im, Hm, 11 + 1000 * rank, dev)
        w2_q, w2_s = quantise_weights_per_channel(el, Hm, Im, 12 + 1000 * rank, dev)
        g = torch.Generator().manual_seed(21)
        x = torch.randn((Mm, Hm), generator=g, dtype=torch.float32).to(torch.bfloat16)
        logits = torch.randn((Mm, Em), generator=g, dtype=torch.float32).to(dev)
        tw, ti = aiter_b200.fused_topk(x.to(dev), logits, Km, True)
        ml = Mm // world
        rows = slice(rank * ml, (rank + 1) * ml)
        dx, dtw, dti = x[rows].to(dev), tw[rows].contiguous(), ti[rows].contiguous()
        if world == 1:
            fn = lambda: aiter_b200.fused_moe(dx, w1_q, w2_q, dtw, dti, quant_type=QT.per_Token, w1_scale=w1_s, w2_scale=w2_s)
        else:
            fn = lambda: ep.ep_fused_moe(dx, w1_q, w2_q, dtw, dti, w1_s, w2_s, Em, exchange="nccl", quant_type=QT.per_Token)
        ms = max_over_ranks(median_ms(fn, sync, steps))
        out["cfg3_mixtral_per_token_M4096_H4096_I14336_E8_topk2"] = {
            "ms_per_layer": ms, "tflops": 6.0 * Mm * Km * Hm * Im / (ms * 1e-3) / 1e12,
            "parallelism": f"ep{world}" + (" (nccl exchange)" if world > 1 else "")}
        del w1_q, w1_s, w2_q, w2_s
        torch.cuda.empty_cache()
    # ---- config 4
    Hq, Iq, Eq, Kq = 4096, 1536, 128, 8
    if Eq % world == 0:
        el = Eq // world
        w1_q, w1_s = quantise_weights(el, 2 * Iq, Hq, 31 + 1000 * rank, dev)
        w2_q, w2_s = quantise_weights(el, Hq, Iq, 32 + 1000 * rank, dev)
        sweep = {}
        for Mq in (1, 16, 128, 1024, 16384):
            if Mq % world != 0:
                continue   # every rank owns the same number of rows
            g = torch.Generator().manual_seed(Mq)
            x = torch.randn((Mq, Hq), generator=g, dtype=torch.float32).to(torch.bfloat16)
            tw, ti = zipf_routing(Mq, Eq, Kq, Mq)
            ml = Mq // world
            rows = slice(rank * ml, (rank + 1) * ml)
            dx, dtw, dti = x[rows].to(dev), tw[rows].to(dev), ti[rows].to(dev)
            if world == 1:
                fn = lambda: aiter_b200.fused_moe(dx, w1_q, w2_q, dtw, dti, quant_type=QT.per_1x128, w1_scale=w1_s, w2_scale=w2_s)
            else:
                fn = lambda: ep.ep_fused_moe(dx, w1_q, w2_q, dtw, dti, w1_s, w2_s, Eq, exchange=exchange)
            ms = max_over_ranks(median_ms(fn, sync, steps))
            sweep[str(Mq)] = {"us_per_layer": ms * 1e3, "tflops": 6.0 * Mq * Kq * Hq * Iq / (ms * 1e-3) / 1e12}
        out["cfg4_qwen3_zipf1.2_H4096_I1536_E128_topk8"] = {
            "sweep_M": sweep, "parallelism": f"ep{world}" + (f" ({exchange} exchange)" if world > 1 else "")}
        del w1_q, w1_s, w2_q, w2_s
        torch.cuda.empty_cache()
    aiter_b200.check_device_status()
    return out


def ep_parity_check(out_local, x, tw, ti, w, table, rank, world, dev, n_rows=4):
    """N > 1: the first rows of rank 0's output against the CPU oracle. ``x``, ``tw``, ``ti`` are RANK 0's rows on every
    rank (all ranks must walk the same expert list); ``out_local`` is the caller's own output and is read on rank 0
    only. The experts those rows are routed to are fetched from the ranks that own them (broadcasts, outside every
    timed region); the oracle then runs on rank 0."""
    import torch.distributed as dist
    w1_q, w1_s, w2_q, w2_s = w
    rows_ids = ti[:n_rows]
    needed = sorted(set(int(e) for e in rows_ids.flatten().tolist()))
    owned = [torch.nonzero(table == r).flatten().tolist() for r in range(world)]
    got = []
    for gexp in needed:
        owner = int(table[gexp])
        li = owned[owner].index(gexp)
        parts = []
        for t in (w1_q, w1_s, w2_q, w2_s):
            buf = t[li].contiguous() if rank == owner else torch.empty_like(t[0])
            dist.broadcast(buf.view(torch.uint8), src=owner)   # as bytes: the collective need not know e4m3
            if rank == 0:
                parts.append(buf.cpu())
        got.append(parts)
    if rank != 0:
        return None
    from oracle import moe_oracle
    remap = {gexp: i for i, gexp in enumerate(needed)}
    ids = torch.tensor([[remap[int(e)] for e in row] for row in rows_ids.tolist()], dtype=torch.int32)
    stack = lambda k: torch.stack([p[k] for p in got])
    ref = moe_oracle.fused_moe_ref(x[:n_rows], stack(0), stack(1), stack(2), stack(3), tw[:n_rows], ids)
    st = moe_oracle.error_stats(out_local[:n_rows].cpu(), ref)
    keep = ("numel", "n_diff", "n_one_ulp", "max_abs_over_rms", "max_abs_excl_one_ulp_over_rms", "frac_within", "has_nan")
    res = {k: st[k] for k in keep}
    res["rows"] = n_rows
    res["experts_fetched"] = len(needed)
    res["ok"] = bool((not st["has_nan"]) and st["frac_within"] >= 0.995 and st["max_abs_excl_one_ulp_over_rms"] <= 0.02
                     and st["max_abs_over_rms"] <= 0.04)
    return res


def emit(line):
    """The one JSON line goes to the real stdout; everything else this process (or a library such as NCCL,
    which prints a version banner) writes to stdout has been pointed at stderr."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = os.dup(1)
os.dup2(2, 1)


def main():
    global M_PREFILL, E, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tokens", type=int, default=M_PREFILL, help="override M (profiling a small case)")
    ap.add_argument("--experts", type=int, default=E, help="override E (profiling a small case)")
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--skip-other-configs", action="store_true", help="leave out configs 3 and 4 (other_configs)")
    ap.add_argument("--ep-exchange", default="auto", choices=["auto", "nccl", "p2p"],
                    help="N>1: NCCL all-gather + fp32 reduce-scatter, or dispatch/combine over peer memory; auto = "
                         "peer memory if every rank can map its peers' buffers, else NCCL")
    ap.add_argument("--ep-placement", default="balanced", choices=["contiguous", "balanced", "lpt"],
                    help="N>1: experts in contiguous slices per rank, or placed by the route counts of a calibration "
                         "batch (other seed) so that every rank gets the same number of experts and a level load: "
                         "balanced = the fewest experts exchanged between the slices, lpt = greedy from scratch")
    ap.add_argument("--ep-push-ranges", type=int, default=2,
                    help="N>1, peer-memory exchange: stage 2 in this many column ranges, the push of a finished range "
                         "beside the GEMM of the next (1 = one stage-2 launch, then one push)")
    ap.add_argument("--ep-graph", default="auto", choices=["auto", "on", "off"],
                    help="N>1: replay the expert-parallel layer call from a captured CUDA graph (one driver call per "
                         "step instead of ~14 launches from Python); auto = on, falling back to eager launches on "
                         "all ranks if the capture fails on any")
    ap.add_argument("--cuda-profiler-range", action="store_true",
                    help="bracket the device-timed steps with cudaProfilerStart/Stop (ncu --profile-from-start off)")
    ap.add_argument("--library-fp8-gemm-only", type=int, default=0, metavar="N",
                    help="run nothing but the vendor library's dense e4m3 GEMM (N^3) and print its rate: the known "
                         "workload a profiler's tensor-pipe counters are calibrated on")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.library_fp8_gemm_only:
        n = args.library_fp8_gemm_only
        tf = library_fp8_gemm_tflops(torch.device("cuda", 0), n=n, iters=5)
        print(json.dumps({"library_fp8_gemm": f"torch._scaled_mm {n}^3 e4m3, tensor-wise scales, bf16 out",
                          "tflops": tf, "flops_per_launch": 2.0 * n ** 3}))
        return
    args.warmup = max(args.warmup, 3)
    small = args.tokens != M_PREFILL or args.experts != E
    if small:
        M_PREFILL, E = args.tokens, args.experts
        WORKLOAD = f"small_case_M{M_PREFILL}_H{H}_I{I}_E{E}_topk{TOPK} (not the headline workload)"

    import importlib
    import torch.distributed as dist
    import aiter_b200
    from aiter_b200 import _lib, ep
    fm = importlib.import_module("aiter_b200.fused_moe")
    QT = aiter_b200.QuantType

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # N > 1: several ranks share the host; each stays on the cores (and memory) of its GPU's NUMA node. N = 1 keeps
    # all cores: the CPU baseline leg of that line uses them.
    cpu_affinity = bind_near_gpu(local_rank) if world > 1 else None
    if world > 1:
        import datetime
        # a collective that not every rank reaches ends with an error after this time instead of hanging the job
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    w1_q, w1_s, w2_q, w2_s = make_layer(dev, rank, world)
    x, tw, ti = make_tokens(M_PREFILL, device=dev)
    m_local = M_PREFILL // world
    rows = slice(rank * m_local, (rank + 1) * m_local)
    # pinned host copies of this rank's step inputs, and a pinned landing buffer for its output
    hx, htw, hti = (t[rows].contiguous().pin_memory() for t in (x, tw, ti))
    hout = torch.empty((m_local, H), dtype=torch.bfloat16).pin_memory()
    hout2 = [hout, torch.empty((m_local, H), dtype=torch.bfloat16).pin_memory()]
    dx, dtw, dti = hx.to(dev), htw.to(dev), hti.to(dev)

    # expert -> rank table: contiguous slices, or levelled by the route counts of a calibration batch (another seed),
    # as a loader would place experts from routing statistics; rank r holds its experts in ascending global id
    table = torch.arange(E, dtype=torch.int32) // (E // world)
    placement_info = None
    if world > 1 and args.ep_placement != "contiguous":
        _xc, _twc, tic = make_tokens(M_PREFILL, seed=100, device=dev, bias=router_inputs(M_PREFILL)[2])
        table = ep.balanced_expert_placement(torch.bincount(tic.flatten().long(), minlength=E), world,
                                             method="swap" if args.ep_placement == "balanced" else "lpt")
    if world > 1:
        counts = torch.bincount(ti.flatten().long(), minlength=E)
        load = torch.zeros(world, dtype=torch.long).index_add_(0, table.long(), counts)
        ranks_per_token = torch.zeros((M_PREFILL, world), dtype=torch.bool).scatter_(1, table[ti.long()].long(), True).sum(1)
        placement_info = {"kind": args.ep_placement, "routes_per_rank": load.tolist(),
                          "max_over_mean": float(load.max()) / (float(load.sum()) / world),
                          "mean_ranks_per_token": float(ranks_per_token.float().mean())}
    xr = table.to(dev) if (world > 1 and args.ep_placement != "contiguous") else None

    exchange = args.ep_exchange
    if world > 1 and exchange == "auto":
        try:
            ep.PeerExchange.get(None, m_local, H, dev)   # collective; fails on all ranks or on none
            exchange = "p2p"
        except RuntimeError as e:
            print(f"[bench] peer-memory exchange not available ({e}); using NCCL", file=sys.stderr)
            exchange = "nccl"
    if world == 1:
        def layer(a, b, c):
            return aiter_b200.fused_moe(a, w1_q, w2_q, b, c, quant_type=QT.per_1x128, w1_scale=w1_s, w2_scale=w2_s)
    else:
        ranges = args.ep_push_ranges if exchange == "p2p" else 1

        def layer(a, b, c):
            return ep.ep_fused_moe(a, w1_q, w2_q, b, c, w1_s, w2_s, E, exchange=exchange, expert_rank=xr,
                                   overlap_chunks=ranges)

    eager_layer, captured, cap_dec = layer, None, None
    if world > 1 and args.ep_graph != "off":
        from aiter_b200.graph import CapturedLayer
        err = None
        try:
            captured = CapturedLayer(eager_layer, dx, dtw, dti)
        except Exception as e:   # noqa: BLE001 - any failure means "launch eagerly", agreed on by all ranks below
            err = f"{type(e).__name__}: {e}"
        ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            if args.ep_graph == "on":
                raise RuntimeError(f"--ep-graph on: capture failed ({err or 'on another rank'})")
            print(f"[bench] rank {rank}: graph capture not used ({err or 'failed on another rank'})", file=sys.stderr)
            captured = None
        else:
            def layer(a, b, c):
                # new inputs are copied into the captured tensors; the result is the captured output tensor, which the
                # next replay overwrites (the end-to-end loop copies it out first)
                return captured(a, b, c)

    def step_dev():
        # inputs resident in HBM: with a captured graph they are the captured input tensors themselves
        return captured.replay() if captured is not None else layer(dx, dtw, dti)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world == 1:
        fm.kernel_bench_events = []   # per-kernel event marks of the timed steps (warm-up marks are dropped below)
    t_dev = timed(step_dev, args.steps, args.warmup, sync, profile=args.cuda_profiler_range)
    stage_marks, fm.kernel_bench_events = fm.kernel_bench_events, None
    t_e2e_total = timed_e2e_pipelined(layer, (hx, htw, hti), hout2, dev, args.steps, min(args.warmup, 3), sync,
                                      static_out=captured is not None)
    # the two host copies of a step timed alone (what bounds e2e when they are slower than the layer)
    def copy_ms(pairs, reps=3):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for dst, src in pairs:
                dst.copy_(src, non_blocking=True)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / reps
    h2d_ms = max_over_ranks(copy_ms([(dx, hx), (dtw, htw), (dti, hti)]))
    d2h_ms = max_over_ranks(copy_ms([(hout, step_dev())]))
    launches0 = _lib.launch_count
    eager_layer(dx, dtw, dti)   # a graph replay issues the same kernels without passing the counter
    gpu_launches = (_lib.launch_count - launches0) * args.steps * 2   # device-timed and end-to-end loops
    clocks = sampler.stop() if rank == 0 else None
    aiter_b200.check_device_status()

    ms_step = max_over_ranks(sum(t_dev)) / args.steps
    ms_e2e = max_over_ranks(t_e2e_total) / args.steps
    value = flops(M_PREFILL) / (ms_step * 1e-3) / 1e12
    e2e_value = flops(M_PREFILL) / (ms_e2e * 1e-3) / 1e12

    pk = peaks()
    fp8_peak = 2.0 * pk["bf16_tflops"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 in/out)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens": M_PREFILL, "model_dim": H, "inter_dim": I, "experts": E,
                   "topk": TOPK, "parallelism": f"ep{world}" + (f" ({exchange} exchange, {args.ep_placement} expert placement, "
                                                                f"{'CUDA-graph replay' if captured is not None else 'eager launches'}"
                                                                + (f", push in {ranges} column ranges beside stage 2" if ranges > 1 else "") + ")"
                                                                if world > 1 else ""),
                   "l2_policy": "inputs larger than L2 (11.3 GB of weights per step)"},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(hx.numel() * 2 + htw.numel() * 4 + hti.numel() * 4) * world,
                "d2h_bytes_per_step": int(hout.numel() * 2) * world,
                "h2d_ms_alone": round(h2d_ms, 4), "d2h_ms_alone": round(d2h_ms, 4),
                "how": "pinned host -> device copy of x, topk_weight, topk_ids and device -> pinned host copy of the bf16 "
                       "result every step, on two copy streams overlapping the neighbouring steps' compute"},
        "clocks": clocks,
        "gpu_launches": gpu_launches,   # kernels of this library launched by this rank inside the two timed loops
    }
    if placement_info is not None:
        line["expert_placement"] = placement_info
    if cpu_affinity is not None:
        line["cpu_affinity_rank0"] = cpu_affinity

    if world == 1:
        # per-kernel device time averaged over the timed steps themselves (events recorded inside the timed loop)
        per_call = len(stage_marks) // (args.steps + args.warmup)
        kb_acc = {}
        for c in range(args.warmup, args.steps + args.warmup):
            marks = stage_marks[c * per_call:(c + 1) * per_call]
            for (n0, e0), (_n1, e1) in zip(marks[:-1], marks[1:]):
                kb_acc.setdefault(n0, []).append(e0.elapsed_time(e1))
        kb = {k: sum(v) / len(v) for k, v in kb_acc.items()}
        line["kernels_ms"] = {k: round(v, 4) for k, v in kb.items()}
        s1 = 4.0 * M_PREFILL * TOPK * H * I / (kb["stage1"] * 1e-3) / 1e12
        s2 = 2.0 * M_PREFILL * TOPK * H * I / (kb["stage2"] * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "kernel": "stage-1 GEMM (gate/up + SiLU*up + requant)", "achieved": s1,
                            "peak": fp8_peak, "unit": "TFLOP/s", "frac": s1 / fp8_peak,
                            "traffic": STAGE1_DRAM_BYTES_PER_EXPERT * E if M_PREFILL == 8192 else None,
                            "traffic_source": "extrapolated: " + STAGE1_DRAM_CAPTURE + ", scaled by the expert count",
                            "algorithmic_bytes": 2 * E * I * H + M_PREFILL * H + M_PREFILL * TOPK * I,
                            "peak_source": f"2 x bf16_tflops of {pk['source']} ({pk['bf16_tflops']} TFLOP/s burst); "
                                           "the driver's peak file has no FP8 entry",
                            "stage2_achieved": s2, "stage2_frac": s2 / fp8_peak}
        line["layer_frac_of_fp8_peak"] = value / fp8_peak
        lib = library_fp8_gemm_tflops(dev)
        if lib is not None:
            line["roofline"]["library_fp8_gemm_tflops"] = lib
            line["roofline"]["frac_of_library_fp8_gemm"] = s1 / lib
    if world > 1:
        accb = {}
        for _ in range(5):
            timers = []
            ep.ep_fused_moe(dx, w1_q, w2_q, dtw, dti, w1_s, w2_s, E, timers=timers, exchange=exchange, expert_rank=xr)
            sync()
            for (n0, e0), (_n1, e1) in zip(timers[:-1], timers[1:]):
                accb.setdefault(n0, []).append(e0.elapsed_time(e1))
        line["ep_breakdown_ms_rank0"] = {k: round(sum(v) / len(v), 4) for k, v in accb.items()}
        # the same marks of every rank for the parts that depend on the rank's load: who is the slowest, who waits
        mine_ms = torch.tensor([sum(accb[k]) / len(accb[k]) for k in ("stage1", "stage2", "ep_push", "ep_barrier")],
                               dtype=torch.float32, device=dev)
        all_ms = torch.empty((world, 4), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(all_ms, mine_ms)
        line["ep_ms_per_rank"] = {k: [round(float(v), 4) for v in all_ms[:, i].tolist()]
                                  for i, k in enumerate(("stage1", "stage2", "ep_push", "ep_barrier"))}
        # host time of one layer call (launches only, no synchronisation): what bounds the step when the device is faster
        torch.cuda.synchronize()
        th = []
        for _ in range(5):
            t0 = time.perf_counter()
            step_dev()
            th.append((time.perf_counter() - t0) * 1e3)
            torch.cuda.synchronize()
        line["host_ms_per_call_rank0"] = round(statistics.median(th), 4)
        # Roofline of the sharded layer: the slower of (this rank's share of the flops at the FP8 peak) and (the bytes
        # that must cross NVLink per rank at the measured 770 GB/s per direction); achieved = the step time.
        touched = torch.zeros((M_PREFILL, world), dtype=torch.bool)
        touched.scatter_(1, table[ti.long()].long(), True)                  # [token, rank]: a route on that rank
        owner = torch.arange(M_PREFILL) // m_local
        remote = touched.clone()
        remote[torch.arange(M_PREFILL), owner] = False                      # rows that leave the owning rank
        kb = H // 128
        if exchange == "p2p":
            disp = remote.sum(1)[owner == 0].sum().item() * (H + kb * 4)    # rank 0 sends its rows to the ranks that need them
            comb = remote[:, 0].sum().item() * H * 4                        # rank 0 pushes the partial rows it produced
        else:
            disp = (world - 1) * m_local * (H + kb * 4 + 8 * TOPK)          # all-gather: every rank receives the others' rows
            comb = (world - 1) * m_local * H * 4                            # reduce-scatter of fp32 partials
        t_flops = flops(M_PREFILL) / world / (fp8_peak * 1e12) * 1e3
        t_link = (disp + comb) / 770e9 * 1e3
        line["roofline"] = {"bound": "tensor" if t_flops >= t_link else "nvlink", "achieved": value / world,
                            "peak": fp8_peak, "unit": "TFLOP/s per GPU", "frac": max(t_flops, t_link) / ms_step,
                            "traffic": None, "nvlink_bytes_rank0": int(disp + comb),
                            "target_ms": {"flops_at_fp8_peak": t_flops, "nvlink_at_770GBs": t_link},
                            "peak_source": f"2 x bf16_tflops of {pk['source']}; NVLink: 770 GB/s per direction measured on this pool"}
        # numerical check of the path that was just timed (outside the timed region)
        out_chk = step_dev()
        torch.cuda.synchronize()
        # every rank walks the SAME list of experts (those of rank 0's first rows), each broadcast by its owner
        line["parity_check"] = ep_parity_check(out_chk, x[:m_local], tw[:m_local], ti[:m_local], (w1_q, w1_s, w2_q, w2_s),
                                               table, rank, world, dev)

    if not args.skip_decode and not small and M_DECODE % world == 0:
        # ---- decode case (M=64): HBM-bound weight streaming; N > 1: the same expert-parallel path, 64/N rows per rank
        xd, twd, tid = make_tokens(M_DECODE, seed=1, device=dev)
        md = M_DECODE // world
        rd = slice(rank * md, (rank + 1) * md)
        dxd, dtwd, dtid = xd[rd].to(dev), twd[rd].to(dev), tid[rd].to(dev)
        act_per_rank = [int(torch.unique(tid[table[tid.long()] == r]).numel()) for r in range(world)]
        n_act = int(torch.unique(tid).numel())

        def step_decode():
            return eager_layer(dxd, dtwd, dtid)

        td = timed(step_decode, max(args.steps, 20), args.warmup, sync)
        us = max_over_ranks(statistics.median(td) * 1e3)
        # bytes the busiest rank must stream: its active experts' weights (+ activations, negligible)
        gbs = algorithmic_bytes(M_DECODE, max(act_per_rank)) / (us * 1e-6) / 1e9
        dec = {"metric": "DSV3 FP8-blockscale fused_moe us/layer (M=64)", "value": us, "unit": "us",
               "active_experts": n_act, "active_experts_per_rank": act_per_rank,
               "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s (busiest rank)",
                            "frac": gbs / pk["hbm_gbs"], "traffic": None, "peak_source": f"hbm_gbs of {pk['source']}"}}
        if world == 1:
            kbd = kernel_breakdown(fm, (dxd, w1_q, w2_q, dtwd, dtid, None, w1_s, w2_s, None, None, torch.bfloat16))
            dec["kernels_ms"] = {k: round(v, 4) for k, v in kbd.items()}
            # the same layer replayed from a CUDA graph (how serving stacks run decode): no launch gaps
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                step_decode()
            torch.cuda.current_stream(dev).wait_stream(side)
            with torch.cuda.graph(graph):
                step_decode()
            tg = timed(graph.replay, max(args.steps, 20), args.warmup, sync)
            us_graph = statistics.median(tg) * 1e3
            dec["graph_replay_us"] = us_graph
            dec["graph_replay_frac_of_hbm"] = algorithmic_bytes(M_DECODE, n_act) / (us_graph * 1e-6) / 1e9 / pk["hbm_gbs"]
        elif captured is not None:
            cap_dec = CapturedLayer(eager_layer, dxd, dtwd, dtid)   # collective: all ranks capture here
            tg = timed(cap_dec.replay, max(args.steps, 20), args.warmup, sync)
            us_graph = max_over_ranks(statistics.median(tg) * 1e3)
            dec["graph_replay_us"] = us_graph
            dec["graph_replay_frac_of_hbm"] = (algorithmic_bytes(M_DECODE, max(act_per_rank)) / (us_graph * 1e-6) / 1e9
                                               / pk["hbm_gbs"])
        line["decode"] = dec
        aiter_b200.check_device_status()
    if world == 1 and not args.no_cpu_baseline:
        cb = cpu_baseline(n_exp=64)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if not args.skip_other_configs and not small:
        del w1_q, w1_s, w2_q, w2_s
        torch.cuda.empty_cache()
        line["other_configs"] = bench_other_configs(dev, rank, world, sync, max_over_ranks, exchange, min(args.steps, 10))

    if rank == 0:
        emit(line)
        sys.stdout.flush()
    if world > 1:
        # The result is out. Teardown order: captured graphs (they reference the communicator's work), the peer
        # mappings, then the process group; a teardown that does not finish within 30 s ends the process with status 0
        # instead of holding N GPUs until the launcher's limit.
        import threading
        guard = threading.Timer(30.0, os._exit, (0,))
        guard.daemon = True
        guard.start()
        torch.cuda.synchronize()
        dist.barrier()
        for cap in (captured, cap_dec):
            if cap is not None:
                cap.release()
        torch.cuda.synchronize()
        ep.PeerExchange.clear()
        dist.destroy_process_group()
        guard.cancel()


if __name__ == "__main__":
    main()
