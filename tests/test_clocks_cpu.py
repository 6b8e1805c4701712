"""The clock record of the benchmarks against a stand-in for ``nvidia-smi`` (read-only queries; no GPU needed)."""
import os
import stat
import time

from aeris_gb_b200.utils.clocks import ClockSampler

FAKE = """#!/bin/sh
# prints what `nvidia-smi --query-gpu=... --format=csv,noheader,nounits -lms 200` prints: idle, then under load
echo "0, 210, 1965, 95.1, 0x0000000000000001, Not Active, Not Active, Not Active, Not Active"
echo "0, 1965, 1965, 640.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active"
echo "0, 1500, 1965, 991.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
echo "0, 1470, 1965, 998.2, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
sleep 30
"""


def test_clock_sampler_reports_the_median_under_load_and_the_reasons(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    s = ClockSampler(0)
    s.start()
    for _ in range(50):
        if len(s.rows) >= 4:
            break
        time.sleep(0.1)
    rec = s.stop()
    assert rec["samples"] == 4 and rec["sm_max_mhz"] == 1965.0 and rec["power_w_max"] == 998.2
    assert rec["sm_mhz"] == 1500.0            # median of the three samples drawn above 300 W; the idle one is left out
    assert rec["reasons"] == ["sw_power_cap"]


def test_clock_sampler_without_nvidia_smi(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))
    s = ClockSampler(0)
    s.start()
    rec = s.stop()
    assert rec["sm_mhz"] is None and rec["reasons"] == ["nvidia-smi unavailable"]
