"""Packaging for moodist_b200.

    python -m pip install --no-build-isolation .        # compiles the native libraries, then installs
    python -m pip install --no-build-isolation -e .     # development install: libraries are built in the tree

The native code (``libmoodist_b200.so`` with the sm_100a kernels and the host engine, ``_C.so`` with the torch
bindings, ``_serialize.so``) is compiled by ``moodist_b200/_build.py`` with nvcc and ninja; it needs the CUDA
toolkit and the torch that will be used at run time, hence ``--no-build-isolation``.  ``_C.so`` is tied to the
torch version it was built against, as the reference's wheels are (its ``setup.py`` builds one extension per
supported torch version and picks one at import; here the package refuses to import against another torch
with a message that says how to rebuild).
"""

import os
import sys
from pathlib import Path

from setuptools import Command, Distribution, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent
NATIVE = ["libmoodist_b200.so", "_C.so", "_serialize.so"]


def _version() -> str:
    scope: dict = {}
    exec((ROOT / "moodist_b200" / "version.py").read_text(), scope)
    return scope["__version__"]


def _build_native() -> None:
    """Runs the in-tree build (a no-op for what is already up to date: ninja decides)."""
    if os.environ.get("MOODIST_SKIP_NATIVE_BUILD") == "1":
        return
    sys.path.insert(0, str(ROOT))
    try:
        from moodist_b200 import _build
    finally:
        sys.path.pop(0)
    _build.build(with_torch=True, verbose=bool(os.environ.get("MOODIST_BUILD_VERBOSE")))
    missing = [n for n in NATIVE if not (ROOT / "moodist_b200" / n).exists()]
    if missing:
        raise RuntimeError(f"native build finished without producing {missing}")


class BinaryDistribution(Distribution):
    """The wheel carries compiled libraries: it is specific to this platform, Python and torch."""

    def has_ext_modules(self):
        return True


class BuildNative(Command):
    """``python setup.py build_native``: compile the libraries into the source tree and stop."""

    description = "compile libmoodist_b200.so, _C.so and _serialize.so in the tree"
    user_options: list = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPyWithNative(build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    name="moodist_b200",
    version=_version(),
    description="Collectives, fused collective GEMMs, queues, resharding and sharded training for B200 (sm_100a)",
    long_description=(ROOT / "README.md").read_text(),
    long_description_content_type="text/markdown",
    packages=["moodist_b200", "moodist_b200.models", "moodist_b200.ops", "moodist_b200.parallel", "moodist_b200.utils"],
    package_data={"moodist_b200": NATIVE},
    include_package_data=False,
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_native": BuildNative, "build_py": BuildPyWithNative},
    zip_safe=False,
    distclass=BinaryDistribution,
)
