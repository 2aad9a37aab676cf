"""The host-side pieces of bench.py that run without a GPU: the CPU leg that times the reference's ggml build (here its
bounded-sample form, which a host short of memory falls back to), the memory probe that chooses between the two forms,
and the arithmetic of the roofline object."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_memory_probe_and_in_step_estimate():
    import bench
    assert bench.host_memory_available() > 0
    e = bench.in_step_estimate(3.926e9, 3.0, 6.0, 4.0, 6548.8)
    assert abs(e["ms"] - 2.0) < 1e-9 and abs(e["achieved"] - 1963.0) < 1e-6 and abs(e["frac"] - 1963.0 / 6548.8) < 1e-9
    assert bench.in_step_estimate(1.0, 0.0, 6.0, 4.0, 6548.8)["frac"] is None


def test_cpu_leg_falls_back_to_the_bounded_sample(ref, monkeypatch):
    """With little host memory the CPU leg times one decoder layer and the output projection and says so; the whole-step
    form needs about 23 GB and is what the benchmark box runs."""
    import bench
    from tensorlisp_b200.programs import DecoderConfig
    monkeypatch.setattr(bench, "host_memory_available", lambda: 4 << 30)
    r = bench.cpu_reference_step(DecoderConfig(), time_limit_s=0.0, steps=1, warmup=0)
    assert r["whole_step"] is False and r["kind"] == "reference" and r["sample"].startswith("BOUNDED SAMPLE")
    assert r["value"] > 0 and abs(r["value"] - 32 / (r["ms_per_step"] * 1e-3)) < 1e-6
