"""Builds and runs the stand-alone C++ self-tests of the torch-free core against libmoodist_b200.so:
wire-format golden bytes, registered-memory bounds checks, the bootstrap ring, CPU reduce loops, and the
host engine with ranks as threads of one process."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "moodist_b200")


def _build(name, tmp_path):
    exe = str(tmp_path / name)
    cmd = ["/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++", "-std=c++20", "-O1", "-g",
           f"-I{ROOT}/moodist_b200/csrc", "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "native", name + ".cc"),
           "-o", exe, f"-L{LIBDIR}", "-lmoodist_b200", f"-Wl,-rpath,{LIBDIR}", "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    return exe


def test_core_selftest(tmp_path):
    import moodist_b200  # noqa: F401 - the library must be built

    exe = _build("core_selftest", tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "CORE SELFTEST OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("world,n", [(2, 1000), (4, 20000), (8, 100000), (5, 7)])
def test_engine_selftest(tmp_path, world, n):
    import moodist_b200  # noqa: F401

    exe = _build("engine_selftest", tmp_path)
    r = subprocess.run([exe, str(world), str(n)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ENGINE SELFTEST OK" in r.stdout, r.stdout + r.stderr


def test_topology_binding_on_any_host():
    """The binding answers on hosts without NVML too (an empty GPU table and this machine's boot id)."""
    from moodist_b200._core import _C

    t = _C.topology()
    assert t["node_id"] and isinstance(t["gpus"], list) and len(t["links"]) == len(t["gpus"])
    assert "GPU(s)" in t["text"]
    assert isinstance(_C.numa_cpus(0), list)
