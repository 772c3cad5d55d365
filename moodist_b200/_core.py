"""Loads the native extension modules.

The reference picks one of several ``_C`` builds by torch version (``py/moodist/_core.py:13-27``) and
tolerates missing optional symbols by exposing them as ``None`` (``:30-36``).  Here exactly one torch
build is targeted; the extension is built in-tree (``python moodist_b200/_build.py``) and a missing
build is an ImportError with the fix spelled out, never a silent fallback.
"""

from __future__ import annotations

import importlib
import os

import torch
import torch.distributed  # registers c10d's pybind types, which _C's classes derive from

_HERE = os.path.dirname(os.path.abspath(__file__))


def _load(name: str):
    path = os.path.join(_HERE, name + ".so")
    if not os.path.exists(path):
        raise ImportError(
            f"moodist_b200: native library {name}.so has not been built; run `python moodist_b200/_build.py`"
        )
    return importlib.import_module("moodist_b200." + name)


_C = _load("_C")

MoodistProcessGroup = _C.MoodistProcessGroup
MoodistBackend = _C.MoodistBackend
TcpStore = getattr(_C, "TcpStore", None)
cuda_copy = _C.cuda_copy
set_prefer_kernel_less = _C.set_prefer_kernel_less

# Stores that are still alive when the interpreter exits (held by a reference cycle, a module global, an exception's
# traceback) leave through the coordinated shutdown all the same: a rank that just disappears takes the answers
# it had queued for its peers with it.
if hasattr(_C, "_shutdown_all_stores"):
    import atexit

    atexit.register(_C._shutdown_all_stores)

_serialize = _load("_serialize")


def serialize(obj) -> torch.Tensor:
    """Serialize a Python object into a uint8 tensor (the reference's ``moodist.serialize``,
    ``wrapper/serialize_wrapper.cc:58-118``). The tensor aliases the packed buffer; no copy is made."""
    buf = _serialize.pack(obj)
    if len(buf) == 0:  # cannot happen (every value has a tag byte), kept for torch.frombuffer's sake
        return torch.empty(0, dtype=torch.uint8)
    return torch.frombuffer(buf, dtype=torch.uint8)


def deserialize(tensor: torch.Tensor):
    """Inverse of :func:`serialize`; accepts any CPU uint8 tensor (or bytes-like object)."""
    if isinstance(tensor, torch.Tensor):
        if tensor.dtype != torch.uint8:
            raise TypeError("moodist.deserialize expects a uint8 tensor")
        tensor = tensor.detach().cpu().contiguous().numpy()
    return _serialize.unpack(tensor)


LIB_PATH = os.path.join(_HERE, "libmoodist_b200.so")
