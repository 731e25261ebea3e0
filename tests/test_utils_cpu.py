"""Host-side utilities: the clock sampler against a stand-in `nvidia-smi`, the phase timers without a GPU."""
import os
import stat
import time

import pytest
import torch

from dion_b200.utils.clocks import ClockSampler
from dion_b200.utils.timers import PhaseTimers

_FAKE = """#!/bin/sh
# prints what `nvidia-smi --query-gpu=... --format=csv,noheader,nounits -lms N` prints, forever
i=0
while true; do
  if [ $i -lt 2 ]; then echo "0, 345, 1965, 180.5, Not Active, Not Active, Not Active, Not Active";
  else echo "0, 1650, 1965, 951.2, Not Active, Not Active, Not Active, Active"; fi
  i=$((i+1))
  sleep 0.02
done
"""


def test_clock_sampler_reports_clocks_under_load_and_reasons(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(_FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    s = ClockSampler(gpu_index=0, period_ms=20)
    s.start()
    time.sleep(0.5)
    out = s.stop()
    assert out["samples"] >= 5
    assert out["sm_mhz"] == 1650.0            # the idle samples (low power) do not count
    assert out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    assert out["power_w_max"] == 951.2


def test_clock_sampler_without_the_tool(monkeypatch, tmp_path):
    monkeypatch.setenv("PATH", str(tmp_path))
    s = ClockSampler()
    s.start()
    assert s.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason="describes the machine without a GPU")
def test_phase_timers_are_inert_without_a_gpu():
    t = PhaseTimers(enabled=True)
    t.start("a")
    t.stop("a")
    assert t.summary() == {} and t.max_over_ranks() == {}
