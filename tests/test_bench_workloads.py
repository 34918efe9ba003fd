"""bench.py pieces that need no GPU: the reference arm's answer, the synthetic workloads of the four serving
configurations, and the virtual clock behind the Poisson arrivals."""
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_reports_unavailable_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps",
                        "2", "--warmup", "1"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-500:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line.get("unavailable"), str) and line["unavailable"]


def test_workloads_follow_the_named_distributions():
    b = _bench()
    prompts, outs, arrivals = b.make_workload("llama-2-7b", 1000, 0, 32000)
    pl = np.array([len(p) for p in prompts])
    assert len(prompts) == 1000 and pl.min() >= 4 and pl.max() <= 2048 and 150 < np.median(pl) < 260
    assert min(outs) >= 4 and max(outs) <= 1024 and 130 < np.median(outs) < 240
    assert all(3 <= t < 32000 for t in prompts[0]) and set(arrivals) == {0.0}

    prompts, outs, arrivals = b.make_workload("llama-3-70b", 512, 0, 128256)
    pl = np.array([len(p) for p in prompts])
    assert pl.min() >= 32 and pl.max() <= 8192 and 800 < np.median(pl) < 1300
    assert min(outs) >= 16 and max(outs) <= 2048
    gaps = np.diff(arrivals)
    assert (gaps >= 0).all() and 0.09 < gaps.mean() < 0.16  # Poisson, 8 requests per second

    prompts, outs, arrivals = b.make_workload("qwen3-32b-fp8", 800, 0, 151936)
    prefixes = {tuple(p[:4096]) for p in prompts}
    assert len(prefixes) == 8 and set(outs) == {128}
    suffix = np.array([len(p) - 4096 for p in prompts])
    assert suffix.min() >= 128 and suffix.max() <= 512

    prompts, outs, arrivals = b.make_workload("deepseek-v3-fp8", 256, 0, 129280)
    pl = np.array([len(p) for p in prompts])
    assert pl.min() >= 512 and pl.max() <= 4096 and set(outs) == {512}
    # the same seed gives the same workload (the two timed phases run on identically seeded engines)
    again = b.make_workload("deepseek-v3-fp8", 256, 0, 129280)
    assert again[0] == prompts and again[1] == outs


def test_virtual_clock_skips_idle_gaps():
    b = _bench()
    c = b.VirtualClock()
    t0 = c.now()
    c.skip_to(t0 + 100.0)
    assert 99.9 < c.now() - t0 < 101.0
    c.skip_to(t0 + 50.0)  # never backwards
    assert c.now() - t0 > 99.9
