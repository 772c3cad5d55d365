"""Registered-memory allocators.

``enable_cuda_allocator()`` makes every CUDA tensor of the process come out of the symmetric heap (the
VMM range every peer maps), so collectives read tensors in place instead of staging them and NVLS can be
used on them.  Like the reference's ``moodist.enable_cuda_allocator`` it replaces torch's CUDA allocator
and must therefore be called before the first CUDA allocation.  ``symmetric_pool()`` is the scoped
alternative: only allocations made inside the ``with`` block use the heap (through ``torch.cuda.MemPool``),
torch's caching allocator keeps managing everything else.

``enable_cpu_allocator()`` routes CPU tensor storage through the size-class allocator whose regions the
transport registers whole (reference: ``wrapper/allocator_wrapper.cc``, ``wrapper/cpu_allocator_wrapper.cc``).
"""

from __future__ import annotations

import contextlib
import ctypes

import torch

from ._core import LIB_PATH, _C

_enabled = False


def _allocator():
    """The symmetric-heap allocator as torch's allocator object.  It is created natively so that the hooks
    Python's ``CUDAPluggableAllocator`` cannot install are there too: ``Tensor.record_stream`` reaches the heap
    (a block used on a side stream is not handed out again before that stream is done with it) and
    ``getBaseAllocation`` answers."""
    return _C.cuda_allocator()


def enable_cuda_allocator() -> None:
    """Use the symmetric heap for all CUDA allocations of this process (call before any CUDA allocation)."""
    global _enabled
    if _enabled:
        return
    if torch.cuda.is_initialized() and torch.cuda.memory_allocated() > 0:
        raise RuntimeError("enable_cuda_allocator() must be called before the first CUDA allocation of the process")
    _C.enable_cuda_allocator()
    _enabled = True


def cuda_allocator_enabled() -> bool:
    return _enabled


def symmetric_mem_pool() -> "torch.cuda.MemPool":
    """A ``torch.cuda.MemPool`` backed by the symmetric heap, for ``torch.cuda.use_mem_pool``; tensors
    allocated from it stay valid for as long as the pool object is alive."""
    return torch.cuda.MemPool(_allocator())


@contextlib.contextmanager
def symmetric_pool():
    """Allocations inside the block come from the symmetric heap; yields the ``torch.cuda.MemPool``."""
    pool = torch.cuda.MemPool(_allocator())
    with torch.cuda.use_mem_pool(pool):
        yield pool


def cuda_allocator_stats(device: int | None = None) -> dict:
    """Live / cached bytes, cache hits and misses, and mapped heap bytes of a device."""
    if device is None:
        device = torch.cuda.current_device()
    lib = ctypes.CDLL(LIB_PATH)
    out = (ctypes.c_uint64 * 5)()
    lib.mb_cuda_allocator_stats(ctypes.c_int(device), out)
    stats = dict(zip(("live_bytes", "cached_bytes", "hits", "misses", "heap_mapped_bytes"), (int(v) for v in out)))
    lib.mb_cuda_allocator_cross_stream_frees.restype = ctypes.c_uint64
    stats["cross_stream_frees"] = int(lib.mb_cuda_allocator_cross_stream_frees(ctypes.c_int(device)))
    return stats


def enable_cpu_allocator() -> None:
    """CPU tensors allocated from now on live in memory the transport can register region-wise."""
    _C.enable_cpu_allocator()


def cpu_allocator_debug() -> str:
    """Usage of the CPU allocator per size class."""
    return _C.cpu_allocator_debug()
