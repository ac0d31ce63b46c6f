"""The benchmark's clock sampler, against a fake NVML (no GPU): samples taken before the timed region are left
out, the throttle bits map to the names the record uses, and a binding that fails falls back without raising."""
import importlib.util
import os
import sys
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.argv = argv
    return mod


def fake_nvml(clock, mask):
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: None

    def by_uuid(_):
        raise RuntimeError("no such device")
    fake.nvmlDeviceGetHandleByUUID = by_uuid
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetClockInfo = lambda h, c: clock[0]
    fake.nvmlDeviceGetMaxClockInfo = lambda h, c: 1965
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: mask[0]
    fake.nvmlDeviceGetPowerUsage = lambda h: 812000
    return fake


def test_samples_of_the_timed_region_only(monkeypatch):
    clock, mask = [300], [0x8]          # idle clock and a slowdown bit before the region starts
    monkeypatch.setitem(sys.modules, "pynvml", fake_nvml(clock, mask))
    bench = load_bench()
    s = bench.ClockSampler(0, period_s=0.001)
    s.start()
    time.sleep(0.03)
    clock[0], mask[0] = 1950, 0x4
    time.sleep(0.005)
    s.mark()
    time.sleep(0.03)
    rec = s.stop()
    assert rec["source"] == "nvml" and rec["samples"] >= 5
    assert rec["sm_mhz"] == 1950.0 and rec["sm_min_mhz"] == 1950.0 and rec["sm_max_mhz"] == 1965.0
    assert rec["reasons"] == ["sw_power_cap"]
    assert rec["watts_max"] == 812.0


def test_every_throttle_bit_has_its_name(monkeypatch):
    clock, mask = [1200], [0x8 | 0x20 | 0x40 | 0x4 | 0x1]     # 0x1 (idle) is not a slowdown
    monkeypatch.setitem(sys.modules, "pynvml", fake_nvml(clock, mask))
    bench = load_bench()
    s = bench.ClockSampler(0, period_s=0.001)
    s.start()
    s.mark()
    time.sleep(0.02)
    rec = s.stop()
    assert rec["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_power_cap", "sw_thermal_slowdown"]


def test_failing_binding_falls_back_without_raising(monkeypatch):
    broken = types.ModuleType("pynvml")

    def init():
        raise RuntimeError("driver not loaded")
    broken.nvmlInit = init
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    monkeypatch.setenv("PATH", "")          # no nvidia-smi either
    bench = load_bench()
    s = bench.ClockSampler(0)
    s.start()
    s.mark()
    rec = s.stop()
    assert rec["sm_mhz"] is None and rec["reasons"]


def test_fallback_parses_nvidia_smi_lines(monkeypatch, tmp_path):
    """Without the binding the sampler reads `nvidia-smi -lms` lines: a stand-in script prints two of them."""
    broken = types.ModuleType("pynvml")

    def init():
        raise RuntimeError("driver not loaded")
    broken.nvmlInit = init
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "echo '0, 1950, 1965, 512.3, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1935, 1965, 640.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active'\n"
                    "sleep 5\n")
    fake.chmod(0o755)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ.get("PATH", ""))
    bench = load_bench()
    s = bench.ClockSampler(0)
    s.start()
    s.mark()
    time.sleep(0.3)
    rec = s.stop()
    assert rec["source"] == "nvidia-smi" and rec["samples"] == 2
    assert rec["sm_mhz"] == 1942.5 and rec["sm_max_mhz"] == 1965.0
    assert rec["reasons"] == ["sw_power_cap"]
