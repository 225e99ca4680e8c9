"""Host-side pieces of bench.py that do not need a GPU: the clock / throttle sampler against a fake NVML, and the
reference arm's answer."""
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class FakeNvml:
    NVML_CLOCK_SM = 1
    nvmlClocksThrottleReasonSwPowerCap = 0x4
    nvmlClocksThrottleReasonHwSlowdown = 0x8

    def __init__(self):
        self.calls = 0

    def nvmlDeviceGetMaxClockInfo(self, h, kind):
        return 1965

    def nvmlDeviceGetClockInfo(self, h, kind):
        self.calls += 1
        return 1500 + 10 * self.calls

    def nvmlDeviceGetCurrentClocksEventReasons(self, h):
        return 0x4 if self.calls >= 3 else 0x8      # a hardware slowdown only before the mark


def test_clock_sampler_reports_only_the_timed_region():
    b = _bench()
    s = b.ClockSampler(0, period_s=0.02)
    s.nvml, s.handle = FakeNvml(), object()
    s.thread = threading.Thread(target=s._poll, daemon=True)
    s.thread.start()
    time.sleep(0.05)            # start-up phase: these samples carry the hw_slowdown flag
    while s.nvml.calls < 3:
        time.sleep(0.01)
    time.sleep(0.03)
    s.mark()
    time.sleep(0.1)
    out = s.stop()
    assert out["source"] == "nvml" and out["sm_max_mhz"] == 1965.0 and out["samples"] >= 2
    assert out["reasons"] == ["sw_power_cap"]            # the earlier hw_slowdown samples were dropped
    assert out["sm_mhz"] > 1530


def test_reference_arm_prints_unavailable():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True,
                       text=True, timeout=300, env=dict(os.environ, PYTHONPATH=ROOT))
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
