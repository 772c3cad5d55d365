"""moodist.Queue on CPU ranks: local and cross-rank put/get, FIFO order, qsize/empty, non-blocking Empty,
objects, large tensors (pulled with a one-sided read), all ranks into one queue, transactions, multicast
and named queues (the reference's tests/test_queue.py cases plus the 1000 x int64[256] workload)."""

import pickle
import time
from queue import Empty

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _queues(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    q = moodist.Queue(pg, location=0)
    # local put/get on the owner
    if rank == 0:
        q.put_tensor(torch.arange(5))
        assert torch.equal(q.get_tensor(), torch.arange(5))
        assert q.empty() and q.qsize() == 0
        with pytest.raises(Empty):
            q.get_tensor(block=False)
    dist.barrier()
    # cross-rank: the last rank puts 1000 int64[256] tensors, rank 0 reads them in FIFO order
    n = 1000
    if rank == world - 1:
        for i in range(n):
            q.put_tensor(torch.full((256,), i, dtype=torch.int64))
    if rank == 0:
        for i in range(n):
            t = q.get_tensor(timeout=30)
            assert t.dtype == torch.int64 and t.shape == (256,) and int(t[0]) == i and int(t[-1]) == i
    dist.barrier()
    # remote get: rank 0 fills its own queue, the other ranks read from it
    if rank == 0:
        for i in range(3 * (world - 1)):
            q.put_object({"i": i, "from": rank})
    else:
        got = [q.get_object(timeout=30) for _ in range(3)]
        assert all(g["from"] == 0 for g in got)
    dist.barrier()
    assert q.qsize() == 0
    # timeout on an empty remote queue raises Empty and takes about that long
    if rank == world - 1:
        t0 = time.time()
        with pytest.raises(Empty):
            q.get_tensor(timeout=0.3)
        assert 0.25 < time.time() - t0 < 5
    dist.barrier()
    # large tensor (not inlined)
    big = torch.randn(1 << 18)
    if rank == world - 1:
        torch.manual_seed(7)
        w = q.put_tensor(torch.randn(1 << 18))
        w.wait()
    if rank == 0:
        torch.manual_seed(7)
        assert torch.equal(q.get_tensor(timeout=30), torch.randn(1 << 18))
    dist.barrier()
    # every rank puts into one queue
    q.put_object(("hello", rank))
    if rank == 0:
        seen = sorted(q.get_object(timeout=30)[1] for _ in range(world))
        assert seen == list(range(world))
    dist.barrier()
    # transactions: nothing is visible until commit; cancel drops everything
    q2 = moodist.Queue(pg, location=0, name="tx_queue")
    if rank == world - 1:
        with q2.transaction() as tx:
            tx.put_object("a")
            tx.put_object("b")
            time.sleep(0.3)
        try:
            with q2.transaction() as tx:
                tx.put_object("dropped")
                raise KeyError("cancel")
        except KeyError:
            pass
        q2.put_object("c")
    if rank == 0:
        time.sleep(0.1)
        assert q2.qsize() == 0  # the transaction is still open on the sender
        assert [q2.get_object(timeout=30) for _ in range(3)] == ["a", "b", "c"]
    dist.barrier()
    # multicast: one put reaches every location
    qm = moodist.Queue(pg, location=range(world), name="multicast")
    qm.put_object(("mc", rank))
    got = sorted(qm.get_object(timeout=30)[1] for _ in range(world))
    assert got == list(range(world))
    dist.barrier()
    # named queues can be pickled and rebuilt
    clone = pickle.loads(pickle.dumps(q2))
    if rank == 0:
        clone.put_object("via clone")
        assert q2.get_object(timeout=30) == "via clone"
    # wait()
    qw = moodist.Queue(pg, location=0, name="waiter")
    if rank == 0:
        assert qw.wait(timeout=0.1) is False
    dist.barrier()
    if rank == world - 1:
        qw.put_object(1)
    if rank == 0:
        assert qw.wait(timeout=30) is True
        assert qw.get_object() == 1
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_queue(world):
    run_ranks(_queues, world, timeout=180)
