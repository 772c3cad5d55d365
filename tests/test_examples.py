"""The CPU example runs end to end."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_queue_and_reshard_example():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "queue_and_reshard_cpu.py")], capture_output=True,
                       text=True, timeout=180)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
