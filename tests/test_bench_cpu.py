"""Host-side pieces of bench.py that need no GPU: the clock sampler against a stand-in for nvidia-smi."""
import os
import stat
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_clock_sampler_reports_only_samples_inside_the_timed_window(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    # first second: a low clock with a thermal reason (outside the window), afterwards the steady-state line
    fake.write_text("#!/bin/bash\n"
                    "for i in 1 2 3 4 5 6 7 8 9 10; do echo '0, 900, 1965, 300.0, 0x40, Not Active, Active, Not Active, Not Active'; sleep 0.1; done\n"
                    "while true; do echo '0, 1890, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active'; sleep 0.1; done\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    import bench
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(1.4)                      # "warm-up": the query loop is already running
    s.mark_begin()
    time.sleep(0.8)                      # "timed region"
    out = s.stop()
    assert out["sm_mhz"] == 1890.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]          # the thermal samples arrived before the window
    assert 5 <= out["samples"] <= 14 and 0.7 <= out["window_s"] <= 1.2
