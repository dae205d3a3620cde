"""bench.py's host-side arithmetic: the algorithmic bytes behind `roofline.achieved` and the clock record."""
import importlib.util
import os

import pytest


@pytest.fixture(scope="module")
def bench():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    spec = importlib.util.spec_from_file_location("bench_under_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_kernel_bytes_follow_the_shapes(bench):
    from tessera_b200 import synth
    cfg, rows = synth.QWEN3_0_6B, 64
    # weights once (bf16), the launch's rows in, its rows out: n k 2 + m k 2 + out bytes
    assert bench.kernel_bytes("linear_qkv", cfg, rows, 0) == 2 * 4096 * 1024 + 2 * 64 * 1024 + 2 * 64 * 4096
    assert bench.kernel_bytes("linear_gate_up", cfg, rows, 0) == 2 * 6144 * 1024 + 2 * 64 * 1024 + 2 * 64 * 3072
    assert bench.kernel_bytes("linear_o", cfg, rows, 0) == 2 * 1024 * 2048 + 2 * 64 * 2048 + 8 * 64 * 1024
    assert bench.kernel_bytes("linear_down", cfg, rows, 0) == 2 * 1024 * 3072 + 2 * 64 * 3072 + 8 * 64 * 1024
    assert bench.kernel_bytes("linear_unembed", cfg, rows, 0) == 2 * 151936 * 1024 + 2 * 64 * 1024 + 4 * 64 * 151936
    # every visible key and value row once (8 kv heads x 128 x 2 bytes, twice), q in and out
    assert bench.kernel_bytes("attend_rows", cfg, rows, 64 * 170) == 64 * 170 * 4096 + 2 * 64 * 2048 * 2
    assert bench.kernel_bytes("top_1", cfg, rows, 0) == 0.0


def test_clock_record_uses_samples_inside_the_timed_regions(bench):
    s = bench.ClockSampler(0, enabled=False)
    when = s._when("2026/01/02 03:04:05.500")
    assert when is not None and s._when("garbage") is None
    line = lambda stamp, mhz, cap: f"{stamp}, {mhz}, 1965, 700.1, 0x4, Not Active, Not Active, Not Active, {cap}"
    s.lines = [line("2026/01/02 03:04:04.000", 1200, "Not Active"),     # before the region: idle clocks
               line("2026/01/02 03:04:05.400", 1965, "Not Active"),
               line("2026/01/02 03:04:05.600", 1905, "Active"),
               "not a sample"]
    s.windows = [(when - 0.2, when + 0.2)]
    got = s.summary()
    assert got["samples"] == 2 and got["sm_mhz"] == 1935.0 and got["sm_max_mhz"] == 1965.0
    assert got["reasons"] == ["sw_power_cap"] and got["window"] == "timed regions"
    # a region that fell between two samples: the load around it, and the record says so
    s.windows = [(when - 0.01, when + 0.01)]
    got = s.summary()
    assert got["samples"] == 2 and got["window"].startswith("warm-up")
    # nothing sampled at all
    s.lines = []
    assert s.summary()["samples"] == 0
