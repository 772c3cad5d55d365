"""The clock sampler parses what `nvidia-smi` prints (a recorded sample through a stand-in executable), survives a
missing `nvidia-smi`, and never changes a setting (it only ever passes query flags)."""

import os
import stat
import time

from moodist_b200.utils.clocks import ClockSampler

_FAKE = """#!/bin/sh
# stand-in for nvidia-smi: records its arguments, prints a few samples, then idles until terminated
echo "$@" > "$FAKE_SMI_ARGS"
echo "0, 1965, 1965, 180.11, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active"
echo "0, 1305, 1965, 998.20, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
echo "0, 1290, 1965, 999.90, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
echo "0, [N/A], 1965, 999.90, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
echo "garbage line"
exec sleep 30
"""


def test_sampler_parses_recorded_output(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(_FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    args_file = tmp_path / "args.txt"
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")
    monkeypatch.setenv("FAKE_SMI_ARGS", str(args_file))
    s = ClockSampler(3)
    s.start()
    time.sleep(0.5)
    s.stop()
    out = s.summary()
    assert out["samples"] == 3 and out["sm_mhz"] == 1305.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    args = args_file.read_text()
    assert "--query-gpu=" in args and "-i 3" in args
    # read-only: no flag that sets clocks, power limits, persistence or compute mode
    for forbidden in ("-lgc", "-rgc", "-ac", "-rac", "-pl", "-pm", "-c ", "--gpu-reset", "-mig", "-e "):
        assert forbidden not in args, args


def test_sampler_without_nvidia_smi(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))  # nothing there
    s = ClockSampler(0)
    s.start()
    s.stop()
    assert s.summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
