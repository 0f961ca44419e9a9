"""Host-side pieces of bench.py that need no GPU: the clock record and the reference arm's line."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_clock_summary_merges_both_readers():
    c = _bench().ClockSampler("0")
    c.lines = ["0, 1965, 1965, 612.3, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1950, 1965, 640.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
               "garbage"]
    c.nvml_samples = [(1965.0, 1965.0, 0x0), (1965.0, 1965.0, 0x20), (1935.0, 1965.0, 0x1)]
    s = c.summary()
    assert s["samples"] == 5 and s["samples_nvidia_smi"] == 2 and s["samples_nvml"] == 3
    assert s["sm_mhz"] == 1965.0 and s["sm_max_mhz"] == 1965.0
    assert s["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]   # idle (0x1) is not a throttle reason


def test_clock_summary_without_samples():
    s = _bench().ClockSampler("GPU-00000000-0000-0000-0000-000000000000").summary()
    assert s == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


def test_clock_sampler_survives_a_box_without_nvml():
    import time
    with _bench().ClockSampler("0") as c:
        time.sleep(0.02)
    assert c.summary()["samples"] >= 0
