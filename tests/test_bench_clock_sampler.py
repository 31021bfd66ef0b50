"""bench.py's clock sampler against a stand-in for nvidia-smi (a script that takes a while to come up and then
prints one line per period): the sampler is up before the timed region starts, only lines that arrive inside
the region count, a job has one sampler, and a machine without nvidia-smi gives an empty summary."""
import os
import stat
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

FAKE = """#!/bin/sh
sleep 0.3
i=0
while [ $i -lt 200 ]; do
  if [ $i -lt 4 ]; then echo "1200, 1965, Not Active, Not Active, Not Active, Not Active"
  else echo "1800, 1965, Not Active, Not Active, Not Active, Active"; fi
  i=$((i+1))
  sleep 0.05
done
"""


def test_sampler_counts_only_the_timed_region(tmp_path, monkeypatch):
    import bench
    exe = tmp_path / "nvidia-smi"
    exe.write_text(FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    s = bench.ClockSampler(0, period_ms=50)
    t0 = time.perf_counter()
    s.start()
    assert 0.25 < time.perf_counter() - t0 < 2.5 and len(s.rows) >= 1   # waited for the first line, not longer
    time.sleep(0.4)            # "warm-up": the 1200 MHz lines arrive here
    s.begin()
    time.sleep(0.4)
    s.end()
    out = s.summary()
    assert out["samples"] >= 5 and out["sm_mhz"] == 1800.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    assert s.proc.poll() is not None                                       # the stand-in was stopped


def test_disabled_and_missing_sampler_give_an_empty_summary(tmp_path, monkeypatch):
    import bench
    with bench.ClockSampler(0, enabled=False) as s:
        pass
    assert s.proc is None and s.summary()["samples"] == 0 and s.summary()["sm_mhz"] is None
    monkeypatch.setenv("PATH", str(tmp_path))                              # no nvidia-smi anywhere
    with bench.ClockSampler(0) as s2:
        pass
    assert s2.summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
