"""Distributed queues of tensors and Python objects.

    q = moodist.Queue(group, location=0)            # lives on rank 0; every rank may put / get
    q.put_tensor(torch.arange(4))
    q.put_object({"any": "picklable thing"})        # goes through moodist.serialize
    t = q.get_tensor(timeout=1.0)                   # raises queue.Empty when nothing arrives in time
    with q.transaction() as tx:                     # all puts become visible together, or not at all
        tx.put_tensor(a); tx.put_tensor(b)

``location`` may be an iterable of ranks: every item is then delivered to each of them (multicast).  A
queue that has a ``name`` can be rebuilt anywhere in the job from the name of its group, its location and
that name, which is what pickling one does.

The public surface (constructor arguments, method names and their keyword arguments, ``Empty`` on a timed
out ``get``) is that of the reference's ``py/moodist/queue.py``; the native queue behind it is
``csrc/core/queue.cc``.
"""

from __future__ import annotations

from queue import Empty

from ._core import deserialize, serialize
from .backend import find_process_group


def _native_group(group):
    """The native moodist group behind whatever the caller passed: a group name, a moodist group, or a
    ``torch.distributed`` process group that runs on the moodist backend."""
    if isinstance(group, str):
        found = find_process_group(group)
        if found is None:
            raise ValueError(f"no live moodist process group is named {group!r} in this process")
        return found
    if hasattr(group, "Queue") and hasattr(group, "moodist_name"):
        return group
    getter = getattr(group, "_get_backend", None)
    if getter is not None:
        import torch

        for device in ("cpu", "cuda"):
            try:
                native = getter(torch.device(device))
            except RuntimeError:
                continue
            if hasattr(native, "Queue") and hasattr(native, "moodist_name"):
                return native
    raise TypeError(f"moodist.Queue needs a moodist process group (or its name), not {type(group).__name__}")


class Queue:
    """A FIFO that lives on one rank (or, multicast, on several) and that every rank of the group can use."""

    def __init__(self, process_group, location, streaming=False, name=None):
        native = _native_group(process_group)
        self.location = location if isinstance(location, int) else [int(r) for r in location]
        self.streaming = bool(streaming)
        self.process_group_name = native.moodist_name()
        self.impl = native.Queue(location=self.location, streaming=self.streaming, name=name)

    # ---- producers --------------------------------------------------------------------------------
    def put_tensor(self, tensor, *, transaction=0):
        """Queue a tensor.  The returned work object finishes the transfer when it is waited on or dropped."""
        return self.impl.put(tensor, transaction, True)

    def put_object(self, object, *, transaction=0):
        """Queue any Python object ``moodist.serialize`` can encode."""
        return self.impl.put(serialize(object), transaction, False)

    def transaction(self):
        """``with q.transaction() as tx``: the block's puts reach consumers together and in order, or, if the
        block raises, not at all."""
        return TransactionContextManager(self)

    # ---- consumers --------------------------------------------------------------------------------
    def get_tensor(self, block=True, timeout=None, return_size=False):
        item, remaining = self.impl.get(block=block, timeout=timeout)
        if item is None:
            raise Empty
        if return_size:
            return item, remaining
        return item

    def get_object(self, block=True, timeout=None, return_size=False):
        item, remaining = self.get_tensor(block=block, timeout=timeout, return_size=True)
        value = deserialize(item)
        if return_size:
            return value, remaining
        return value

    def qsize(self):
        return self.impl.qsize()

    def empty(self):
        return self.qsize() == 0

    def wait(self, timeout=None):
        """Block until the queue holds something (or ``timeout`` seconds have passed); truthy when it does."""
        return self.impl.wait(timeout=timeout)

    # ---- pickling: a named queue travels as the recipe to look it up again ---------------------------------
    def __reduce__(self):
        return Queue, (self.process_group_name, self.location, self.streaming, self.impl.name())


class TransactionContextManager:
    """Groups puts: begun on entry, committed on a clean exit, cancelled when the block raises."""

    def __init__(self, queue):
        self.queue = queue
        self.id = None

    def __enter__(self):
        self.id = self.queue.impl.transaction_begin()
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        finish = self.queue.impl.transaction_cancel if exc_type is not None else self.queue.impl.transaction_commit
        finish(self.id)
        return False

    def put_tensor(self, tensor):
        return self.queue.put_tensor(tensor, transaction=self.id)

    def put_object(self, object):
        return self.queue.put_object(object, transaction=self.id)
