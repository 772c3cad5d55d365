"""Registration with ``torch.distributed``: backend ``"moodist"`` for CPU and CUDA tensors and the
``moodist://host:port?rank=R&world_size=W`` rendezvous scheme (reference: ``py/moodist/backend.py:15-122``).
"""

from __future__ import annotations

import urllib.parse
from datetime import timedelta

import torch
import torch.distributed

from ._core import MoodistProcessGroup, TcpStore, _C


class PreferKernelLessContext:
    """Sets ``prefer_kernel_less`` on a group; restores the old value when used as a context manager."""

    def __init__(self, pg, value: bool):
        self.pg = pg
        self.old_value = pg.get_prefer_kernel_less()
        pg.set_prefer_kernel_less(bool(value))

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.pg.set_prefer_kernel_less(self.old_value)
        return False


MoodistProcessGroup.prefer_kernel_less = lambda self, value: PreferKernelLessContext(self, value)


def find_process_group(name: str):
    """Look a live moodist group up by its name (``group.moodist_name()``); ``None`` if unknown."""
    return _C.find_process_group(name)


def create_moodist_backend(store: torch.distributed.Store, rank: int, size: int, timeout: timedelta):
    """Creator handed to ``Backend.register_backend``. Groups register themselves by name natively, so
    ``find_process_group`` works for as long as the group object is alive anywhere in the process."""
    return MoodistProcessGroup(store, rank, size)


def get_backend(group=None, device: str | torch.device = "cuda"):
    """The moodist backend object behind a ``torch.distributed`` process group (default: WORLD)."""
    pg = group if group is not None else torch.distributed.distributed_c10d._get_default_group()
    if isinstance(pg, MoodistProcessGroup):
        return pg
    return pg._get_backend(torch.device(device))


def rendezvous_handler(url: str, timeout: timedelta = torch.distributed.distributed_c10d.default_pg_timeout, **kwargs):
    """``init_method="moodist://host:port?rank=R&world_size=W"`` -> a moodist TcpStore."""
    if TcpStore is None:
        raise RuntimeError("moodist TcpStore is not available in this build")
    result = urllib.parse.urlparse(url)
    if result.hostname is None:
        raise ValueError(f"moodist rendezvous URL has no hostname: {url}")
    if result.port is None:
        raise ValueError(f"moodist rendezvous URL has no port: {url}")
    query = urllib.parse.parse_qs(result.query)
    for k in ("rank", "world_size"):
        if k not in query:
            raise ValueError(f"moodist rendezvous URL lacks the '{k}' query parameter: {url}")
    world_size = int(query["world_size"][0])
    rank = int(query["rank"][0])
    yield (TcpStore(result.hostname, result.port, "foo", world_size, rank, timeout), rank, world_size)


if "MOODIST" not in getattr(torch.distributed.Backend, "backend_list", []) and not hasattr(
    torch.distributed.Backend, "MOODIST"
):
    torch.distributed.Backend.register_backend("moodist", create_moodist_backend, devices=("cpu", "cuda"))
if TcpStore is not None:
    try:
        torch.distributed.distributed_c10d.register_rendezvous_handler("moodist", rendezvous_handler)
    except RuntimeError:
        pass  # already registered (module re-import)
