"""The CPU examples run end to end."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_queue_and_reshard_example():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "queue_and_reshard_cpu.py")], capture_output=True,
                       text=True, timeout=180)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


def test_ddp_and_pipeline_example():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "ddp_and_pipeline_cpu.py")], capture_output=True,
                       text=True, timeout=180)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
    assert "replicas identical" in r.stdout and "pipeline of 3 stages: [24.0, 48.0, 72.0, 96.0]" in r.stdout
