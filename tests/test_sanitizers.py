"""The torch-free core under AddressSanitizer (with leak detection), ThreadSanitizer and
UndefinedBehaviorSanitizer: `python moodist_b200/_build.py --sanitize <kind>` builds an instrumented copy of the
library outside the tree, and the stand-alone C++ self-tests (wire format, planner, store mesh, transport, the
host engine with 2-8 ranks as threads doing every CPU collective) run against it.  Any report fails the test.
With `--python` the serializer and the torch bindings are instrumented as well and a Python scenario runs against
that copy of the package.  The reference has the same switches (ENABLE_ASAN / ENABLE_TSAN in its
CMakeLists.txt:6-25)."""

import importlib.util
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _builder():
    spec = importlib.util.spec_from_file_location("_moodist_b200_build", os.path.join(ROOT, "moodist_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("kind", ["address", "undefined", "thread"])
def test_core_selftests_under_sanitizer(kind, tmp_path):
    b = _builder()
    b.build(sanitize=kind)
    libdir = str(b.sanitized_dir(kind))
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1",
               TSAN_OPTIONS="halt_on_error=1:second_deadlock_stack=1")
    for name, runs in (("core_selftest", [[]]), ("engine_selftest", [["2", "1000"], ["5", "7"], ["4", "20000"]])):
        exe = str(tmp_path / f"{name}_{kind}")
        cmd = [cxx, "-std=c++20", "-O1", "-g", f"-fsanitize={kind}", "-fno-omit-frame-pointer", f"-I{ROOT}/moodist_b200/csrc",
               "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "native", name + ".cc"), "-o", exe, f"-L{libdir}",
               "-lmoodist_b200", f"-Wl,-rpath,{libdir}", "-pthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-4000:]
        for args in runs:
            r = subprocess.run([exe] + args, capture_output=True, text=True, timeout=300, env=env)
            out = r.stdout + r.stderr
            assert r.returncode == 0 and "SELFTEST OK" in out, out[-6000:]
            for marker in ("ERROR: AddressSanitizer", "ERROR: LeakSanitizer", "WARNING: ThreadSanitizer", "runtime error:"):
                assert marker not in out, out[-6000:]


def test_python_package_under_address_sanitizer(tmp_path):
    """`_build.py --sanitize address --python` makes an instrumented copy of the whole package (serializer, torch
    bindings and core compiled with AddressSanitizer next to links to the Python sources); a scenario of
    serializer fuzzing and three CPU ranks runs against it in a fresh interpreter with the sanitizer's runtime
    preloaded.  Rank processes inherit the environment, so their native code is checked as well."""
    import sys

    b = _builder()
    b.build(sanitize="address", python=True)
    env = dict(os.environ)
    env.update(b.sanitized_env("address"))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "sanitized_scenario.py"), "200"], cwd=str(tmp_path),
                       capture_output=True, text=True, timeout=1500, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "SCENARIO OK" in out, out[-6000:]
    assert str(b.sanitized_package_dir("address")) in out, out[-2000:]  # the instrumented copy is what ran
    assert "ERROR: AddressSanitizer" not in out, out[-6000:]
