"""Distributed queues of tensors and Python objects (reference: ``py/moodist/queue.py:11-100``).

    q = moodist.Queue(group, location=0)            # lives on rank 0; every rank may put / get
    q.put_tensor(torch.arange(4))
    q.put_object({"any": "picklable thing"})        # goes through moodist.serialize
    t = q.get_tensor(timeout=1.0)                   # raises queue.Empty when nothing arrives in time
    with q.transaction() as tx:                     # all puts become visible together, or not at all
        tx.put_tensor(a); tx.put_tensor(b)

``location`` may be a list of ranks: every item is then delivered to each of them (multicast).  Queues
with a ``name`` can be recreated from (group name, location, name) and so can be pickled.
"""

from __future__ import annotations

from queue import Empty

from ._core import deserialize, serialize
from .backend import find_process_group


class TransactionContextManager:
    def __init__(self, queue):
        self.queue = queue

    def __enter__(self):
        self.id = self.queue.impl.transaction_begin()
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        if exc_type is not None:
            self.queue.impl.transaction_cancel(self.id)
        else:
            self.queue.impl.transaction_commit(self.id)

    def put_tensor(self, tensor):
        return self.queue.put_tensor(tensor, transaction=self.id)

    def put_object(self, object):
        return self.queue.put_object(object, transaction=self.id)


class Queue:
    def __init__(self, process_group, location, streaming=False, name=None):
        if isinstance(process_group, str):
            pg_name = process_group
            process_group = find_process_group(pg_name)
            if process_group is None:
                raise ValueError("The Moodist process group by name '%s' could not be found" % pg_name)
        if not hasattr(process_group, "Queue"):
            # a torch.distributed ProcessGroup whose backend is moodist is fine too
            backend = None
            if hasattr(process_group, "_get_backend"):
                import torch

                try:
                    backend = process_group._get_backend(torch.device("cpu"))
                except RuntimeError:
                    backend = None
            if backend is None or not hasattr(backend, "Queue"):
                raise RuntimeError(
                    "moodist.Queue process_group parameter must be a MoodistProcessGroup, but got %s"
                    % str(type(process_group)),
                )
            process_group = backend
        if not isinstance(location, int):
            location = list(location)
        self.impl = process_group.Queue(location=location, streaming=streaming, name=name)
        self.process_group_name = process_group.moodist_name()
        self.location = location
        self.streaming = streaming

    def __reduce__(self):
        return type(self), (self.process_group_name, self.location, self.streaming, self.impl.name())

    def put_tensor(self, tensor, *, transaction=0):
        return self.impl.put(tensor, transaction, True)  # the work waits for completion when dropped

    def get_tensor(self, block=True, timeout=None, return_size=False):
        r, size = self.impl.get(block=block, timeout=timeout)
        if r is None:
            raise Empty
        return (r, size) if return_size else r

    def put_object(self, object, *, transaction=0):
        return self.impl.put(serialize(object), transaction, False)

    def get_object(self, block=True, timeout=None, return_size=False):
        if return_size:
            tensor, size = self.get_tensor(block=block, timeout=timeout, return_size=True)
            return deserialize(tensor), size
        return deserialize(self.get_tensor(block=block, timeout=timeout))

    def qsize(self):
        return self.impl.qsize()

    def empty(self):
        return self.impl.qsize() == 0

    def wait(self, timeout=None):
        return self.impl.wait(timeout=timeout)

    def transaction(self):
        return TransactionContextManager(self)
