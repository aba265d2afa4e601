"""Host-side pieces of bench.py that need no GPU: the clock sampler's reading of nvidia-smi's output (timestamps, throttle
reasons, samples after the timed region left out), against a stand-in nvidia-smi on PATH."""
import os
import stat
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

FAKE = """#!/usr/bin/env python3
import datetime, sys, time
# prints one CSV line every 50 ms like `nvidia-smi --query-gpu=timestamp,clocks.sm,... --format=csv,noheader,nounits -lms 50`
while True:
    now = datetime.datetime.now().strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    print(f"{now}, 1290, 1965, 998.20, 0x0000000000000004, Not Active, Not Active, Not Active, Active", flush=True)
    time.sleep(0.05)
"""


def test_clock_sampler_reads_timestamps_and_reasons(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    import bench
    s = bench.ClockSampler(0)
    time.sleep(0.6)                      # the "timed region"
    out = s.stop()                       # stop() lets the sampler run on for a quarter of a second: those samples do not count
    assert out["sm_mhz"] == 1290.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    assert 3 <= out["samples"] <= 14, out


def test_clock_sampler_without_nvidia_smi(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))
    import bench
    out = bench.ClockSampler(0).stop()
    assert out["sm_mhz"] is None and out["reasons"] == ["nvidia-smi unavailable"]
