"""bench.py helpers that must degrade quietly on a machine without a GPU or NVML."""

import importlib.util
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_module"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_affinity_hint_never_raises_and_leaves_the_process_alone():
    bench = _bench()
    before = os.sched_getaffinity(0)
    msg = bench.bind_near_gpu(0)
    assert isinstance(msg, str) and msg
    if msg.startswith("unchanged"):
        assert os.sched_getaffinity(0) == before
    else:
        os.sched_setaffinity(0, before)


def test_clock_sampler_reports_a_dict_without_a_gpu():
    bench = _bench()
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.05)
    out = s.stop()
    assert set(out) >= {"sm_mhz", "sm_max_mhz", "reasons"}
