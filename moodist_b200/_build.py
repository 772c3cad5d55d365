"""In-tree build of the native libraries (ninja + g++ + nvcc, sm_100a only).

Three shared objects are produced beside this file:

* ``libmoodist_b200.so`` — torch-free core: host runtime (store, transports, engine, queue, planners,
  allocators, peer-memory mapper) and every CUDA kernel, with a plain C API.
* ``_C.so`` — torch glue: c10d ``Backend``/``Store`` subclasses, allocator hooks, pybind11 bindings.
* ``_serialize.so`` — the Python-object serializer (CPython C API).

The reference builds the same three pieces with CMake (``CMakeLists.txt:150-293``); here a single
torch/CUDA version is targeted so a generated ninja file is enough.  ``python moodist_b200/_build.py``
(re)builds whatever is out of date.
"""

from __future__ import annotations

import sys

# Run as a script, this file's directory lands on sys.path and the package's queue.py would shadow the
# standard library's `queue` for everything imported below.
sys.path[:] = [p for p in sys.path if not p.rstrip("/").endswith("moodist_b200")]

import os
import shutil
import subprocess
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = ROOT.parent / "build" / "native"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> str:
    for c in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if c and os.path.exists(os.path.join(c, "bin", "nvcc")):
            return c
    nvcc = shutil.which("nvcc")
    if nvcc:
        return str(Path(nvcc).resolve().parent.parent)
    raise RuntimeError("nvcc not found")


def _sources(sub: str, exts: tuple[str, ...]) -> list[Path]:
    d = CSRC / sub
    if not d.exists():
        return []
    return sorted(p for p in d.iterdir() if p.suffix in exts)


def _q(s) -> str:
    return str(s).replace(" ", "$ ")


SANITIZERS = ("address", "thread", "undefined")


def generate(with_torch: bool = True, sanitize: str | None = None, python: bool = False) -> Path:
    """Write the ninja file.  ``sanitize`` ("address", "thread" or "undefined") describes a second build of the
    torch-free core with that sanitizer, in ``build/native-<sanitizer>/`` (nothing in-tree is touched): the host
    sources are recompiled with ``-fsanitize=...``, the CUDA objects of the regular build are linked in as they
    are.  The reference has the same switches in its CMake file (``ENABLE_ASAN`` / ``ENABLE_TSAN``,
    ``CMakeLists.txt:6-25, 213-218``)."""
    if sanitize is not None:
        return _generate_sanitized(sanitize, python)
    cuda = _cuda_home()
    BUILD.mkdir(parents=True, exist_ok=True)
    pyinc = sysconfig.get_paths()["include"]

    cxx = os.environ.get("MOODIST_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    common = f"-O2 -g1 -fPIC -std=c++20 -Wall -Wno-unused-function -pthread -I{CSRC} -I{cuda}/include"
    nvcc_flags = (
        " ".join(ARCH_FLAGS)
        + f" -lineinfo -O3 -std=c++17 --expt-relaxed-constexpr -Xcompiler -fPIC -I{CSRC} -I{CSRC}/kernels"
    )
    lines = [
        f"cxx = {cxx}",
        f"nvcc = {cuda}/bin/nvcc",
        f"cflags = {common}",
        f"nvflags = {nvcc_flags}",
        "rule cxx",
        "  command = $cxx $cflags $extra -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule nvcc",
        "  command = $nvcc $nvflags -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        "  command = $cxx -shared -o $out $in $ldflags",
        "",
    ]

    core_objs = []
    for src in _sources("core", (".cc",)):
        obj = BUILD / "core" / (src.stem + ".o")
        lines.append(f"build {_q(obj)}: cxx {_q(src)}")
        core_objs.append(obj)
    for src in _sources("kernels", (".cu",)):
        obj = BUILD / "kernels" / (src.stem + ".o")
        lines.append(f"build {_q(obj)}: nvcc {_q(src)}")
        core_objs.append(obj)
    core_lib = ROOT / "libmoodist_b200.so"
    lines.append(f"build {_q(core_lib)}: link {' '.join(_q(o) for o in core_objs)}")
    lines.append(f"  ldflags = -L{cuda}/lib64 -lcudart_static -lrt -ldl -pthread -Wl,--no-undefined")
    targets = [core_lib]

    ser_srcs = _sources("pyser", (".cc",))
    if ser_srcs:
        objs = []
        for src in ser_srcs:
            obj = BUILD / "pyser" / (src.stem + ".o")
            lines.append(f"build {_q(obj)}: cxx {_q(src)}")
            lines.append(f"  extra = -I{pyinc}")
            objs.append(obj)
        lib = ROOT / "_serialize.so"
        lines.append(f"build {_q(lib)}: link {' '.join(_q(o) for o in objs)}")
        lines.append("  ldflags = -pthread")
        targets.append(lib)

    glue_srcs = _sources("glue", (".cc",))
    if with_torch and glue_srcs:
        import torch
        from torch.utils import cpp_extension

        tinc = " ".join(f"-isystem {p}" for p in cpp_extension.include_paths())
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        extra = (
            f"{tinc} -isystem {pyinc} -D_GLIBCXX_USE_CXX11_ABI={abi} -DTORCH_EXTENSION_NAME=_C "
            "-DTORCH_API_INCLUDE_EXTENSION_H -DUSE_C10D -Wno-deprecated-declarations -Wno-sign-compare"
        )
        objs = []
        for src in glue_srcs:
            obj = BUILD / "glue" / (src.stem + ".o")
            lines.append(f"build {_q(obj)}: cxx {_q(src)}")
            lines.append(f"  extra = {extra}")
            objs.append(obj)
        lib = ROOT / "_C.so"
        lines.append(f"build {_q(lib)}: link {' '.join(_q(o) for o in objs)} | {_q(core_lib)}")
        lines.append(
            f"  ldflags = -L{ROOT} -lmoodist_b200 -L{tlib} -ltorch -ltorch_cpu -ltorch_python -lc10 "
            f"-lc10_cuda -ltorch_cuda -Wl,-rpath,'$$ORIGIN' -Wl,-rpath,{tlib} -pthread"
        )
        targets.append(lib)

    lines.append("default " + " ".join(_q(t) for t in targets))
    path = BUILD / "build.ninja"
    text = "\n".join(lines) + "\n"
    if not path.exists() or path.read_text() != text:
        path.write_text(text)
    return path


def sanitized_dir(sanitize: str) -> Path:
    return BUILD.parent / f"native-{sanitize}"


def sanitized_package_dir(sanitize: str) -> Path:
    """Where the instrumented copy of the Python package lives (``--python``): put it first on ``sys.path``."""
    return sanitized_dir(sanitize) / "pkg"


def sanitized_env(sanitize: str) -> dict:
    """Environment for a Python process that imports the instrumented package: the sanitizer's runtime has to be
    loaded before the interpreter (which is not linked against it), together with libstdc++, whose exception
    entry points the runtime wraps; Python's own small-object allocator is switched off so that the sanitizer sees
    every object."""
    cxx = os.environ.get("MOODIST_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    runtime = {"address": "libasan.so", "thread": "libtsan.so", "undefined": "libubsan.so"}[sanitize]

    def where(lib):
        return subprocess.run([cxx, f"-print-file-name={lib}"], capture_output=True, text=True).stdout.strip()

    env = {
        "LD_PRELOAD": f"{where(runtime)}:{where('libstdc++.so')}",
        "PYTHONMALLOC": "malloc",
        "PYTHONPATH": str(sanitized_package_dir(sanitize)),
        "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=0:exitcode=97",
        "UBSAN_OPTIONS": "print_stacktrace=1:halt_on_error=1:exitcode=97",
        "TSAN_OPTIONS": "exitcode=97",
    }
    return env


def _generate_sanitized(sanitize: str, python: bool = False) -> Path:
    if sanitize not in SANITIZERS:
        raise ValueError(f"unknown sanitizer {sanitize!r}: one of {SANITIZERS}")
    cuda = _cuda_home()
    out = sanitized_dir(sanitize)
    out.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("MOODIST_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    san = f"-fsanitize={sanitize} -fno-omit-frame-pointer"
    if sanitize == "undefined":
        san += " -fno-sanitize-recover=undefined"
    common = f"-O1 -g -fPIC -std=c++20 -Wall -Wno-unused-function -pthread {san} -I{CSRC} -I{cuda}/include"
    lines = [
        f"cxx = {cxx}",
        f"cflags = {common}",
        "rule cxx",
        "  command = $cxx $cflags -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        "  command = $cxx -shared -o $out $in $ldflags",
        "",
    ]
    objs = []
    for src in _sources("core", (".cc",)):
        obj = out / "core" / (src.stem + ".o")
        lines.append(f"build {_q(obj)}: cxx {_q(src)}")
        objs.append(obj)
    # device code is not instrumented: the objects nvcc made for the regular build are reused
    kernel_objs = [BUILD / "kernels" / (src.stem + ".o") for src in _sources("kernels", (".cu",))]
    lib = out / "libmoodist_b200.so"
    lines.append(f"build {_q(lib)}: link {' '.join(_q(o) for o in objs + kernel_objs)}")
    lines.append(f"  ldflags = {san} -L{cuda}/lib64 -lcudart_static -lrt -ldl -pthread")
    targets = [lib]
    if python:
        # The whole package, instrumented: the serializer and the torch bindings compiled with the sanitizer too,
        # next to links to the Python sources, so that `import moodist_b200` from there runs the same code with
        # every native line checked.
        import torch
        from torch.utils import cpp_extension

        pkg = sanitized_package_dir(sanitize) / "moodist_b200"
        pkg.mkdir(parents=True, exist_ok=True)
        for entry in ROOT.iterdir():
            if entry.name in ("csrc", "__pycache__") or entry.suffix == ".so":
                continue
            link = pkg / entry.name
            if link.is_symlink() or link.exists():
                continue
            link.symlink_to(entry)
        pyinc = sysconfig.get_paths()["include"]
        tinc = " ".join(f"-isystem {p}" for p in cpp_extension.include_paths())
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        lines += ["rule cxx_extra", "  command = $cxx $cflags $extra -MMD -MF $out.d -c $in -o $out", "  depfile = $out.d",
                  "  deps = gcc"]
        ser_objs = []
        for src in _sources("pyser", (".cc",)):
            obj = out / "pyser" / (src.stem + ".o")
            lines.append(f"build {_q(obj)}: cxx_extra {_q(src)}")
            lines.append(f"  extra = -I{pyinc}")
            ser_objs.append(obj)
        ser_lib = pkg / "_serialize.so"
        lines.append(f"build {_q(ser_lib)}: link {' '.join(_q(o) for o in ser_objs)}")
        lines.append(f"  ldflags = {san} -pthread")
        glue_extra = (
            f"{tinc} -isystem {pyinc} -D_GLIBCXX_USE_CXX11_ABI={abi} -DTORCH_EXTENSION_NAME=_C "
            "-DTORCH_API_INCLUDE_EXTENSION_H -DUSE_C10D -Wno-deprecated-declarations -Wno-sign-compare"
        )
        glue_objs = []
        for src in _sources("glue", (".cc",)):
            obj = out / "glue" / (src.stem + ".o")
            lines.append(f"build {_q(obj)}: cxx_extra {_q(src)}")
            lines.append(f"  extra = {glue_extra}")
            glue_objs.append(obj)
        core_copy = pkg / "libmoodist_b200.so"
        lines.append("rule copy")
        lines.append("  command = cp -f $in $out")
        lines.append(f"build {_q(core_copy)}: copy {_q(lib)}")
        glue_lib = pkg / "_C.so"
        lines.append(f"build {_q(glue_lib)}: link {' '.join(_q(o) for o in glue_objs)} | {_q(core_copy)}")
        lines.append(
            f"  ldflags = {san} -L{pkg} -lmoodist_b200 -L{tlib} -ltorch -ltorch_cpu -ltorch_python -lc10 "
            f"-lc10_cuda -ltorch_cuda -Wl,-rpath,'$$ORIGIN' -Wl,-rpath,{tlib} -pthread"
        )
        targets += [ser_lib, core_copy, glue_lib]
    lines.append("default " + " ".join(_q(t) for t in targets))
    path = out / "build.ninja"
    text = "\n".join(lines) + "\n"
    if not path.exists() or path.read_text() != text:
        path.write_text(text)
    return path


def build(with_torch: bool = True, verbose: bool = False, sanitize: str | None = None, python: bool = False) -> None:
    """Build (incrementally) all native libraries for sm_100a; with ``sanitize`` the instrumented core as well, and
    with ``python`` an instrumented copy of the whole package (``sanitized_package_dir``, ``sanitized_env``)."""
    generate(with_torch)
    jobs = os.environ.get("MOODIST_BUILD_JOBS", str(os.cpu_count() or 4))
    if sanitize is not None:
        build(with_torch=False, verbose=verbose)  # the CUDA objects come from the regular build
        generate(sanitize=sanitize, python=python)
        cmd = [sys.executable, "-m", "ninja", "-C", str(sanitized_dir(sanitize)), "-j", jobs]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout[-20000:])
            raise RuntimeError(f"{sanitize}-sanitizer build failed")
        return
    cmd = [sys.executable, "-m", "ninja", "-C", str(BUILD), "-j", jobs]
    if verbose:
        cmd.append("-v")
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-20000:])
        raise RuntimeError("native build failed")
    if verbose:
        print(r.stdout)


if __name__ == "__main__":
    san = next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--sanitize=")), None)
    if "--sanitize" in sys.argv:
        san = sys.argv[sys.argv.index("--sanitize") + 1]
    if san:
        build(sanitize=san, verbose="-v" in sys.argv, python="--python" in sys.argv)
        print("built:", sanitized_dir(san) / "libmoodist_b200.so")
        if "--python" in sys.argv:
            print("instrumented package:", sanitized_package_dir(san))
            print("run with:", " ".join(f"{k}={v}" for k, v in sanitized_env(san).items()), "python ...")
    else:
        build(with_torch="--no-torch" not in sys.argv, verbose="-v" in sys.argv)
        print("built:", ", ".join(p.name for p in sorted(ROOT.glob("*.so"))))
