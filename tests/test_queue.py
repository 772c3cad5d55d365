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


def _edges(rank, world, port):
    import gc
    import threading

    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    # several consumer threads on one queue: every item is delivered exactly once
    q = moodist.Queue(pg, location=0, name="threads")
    n = 200
    if rank == 1:
        for i in range(n):
            q.put_object(i)
    if rank == 0:
        got, lock = [], threading.Lock()

        def consume():
            while True:
                try:
                    v = q.get_object(timeout=2)
                except Empty:
                    return
                with lock:
                    got.append(v)

        workers = [threading.Thread(target=consume) for _ in range(4)]
        for t in workers:
            t.start()
        for t in workers:
            t.join()
        assert sorted(got) == list(range(n))
    dist.barrier()
    # a named queue travels inside an object and is usable where it arrives
    inner = moodist.Queue(pg, location=1, name="inner")
    carrier = moodist.Queue(pg, location=0, name="carrier")
    if rank == world - 1:
        carrier.put_object({"reply_to": inner})
    if rank == 0:
        carrier.get_object(timeout=20)["reply_to"].put_object("pong")
    if rank == 1:
        assert inner.get_object(timeout=20) == "pong"
    dist.barrier()
    # an object far larger than what a message carries inline
    big = moodist.Queue(pg, location=0, name="big-object")
    if rank == 1:
        big.put_object({"blob": b"z" * (3 << 20), "numbers": list(range(10000))})
    if rank == 0:
        o = big.get_object(timeout=30)
        assert len(o["blob"]) == 3 << 20 and o["numbers"][-1] == 9999
    dist.barrier()
    # dtype and shape survive: narrow and wide types, bool, complex, 0-d, empty, a non-contiguous view
    dq = moodist.Queue(pg, location=0, name="dtypes")
    kinds = (torch.float16, torch.bfloat16, torch.float64, torch.int8, torch.uint8, torch.bool, torch.int16, torch.int32, torch.complex64)
    tensors = [torch.arange(6).to(dt).view(2, 3) for dt in kinds]
    tensors += [torch.tensor(3.5), torch.empty(0, 4), torch.arange(24.0).view(2, 3, 4)[:, 1]]
    if rank == 1:
        for t in tensors:
            dq.put_tensor(t)
    if rank == 0:
        for t in tensors:
            g = dq.get_tensor(timeout=20)
            assert g.dtype == t.dtype and g.shape == t.shape and torch.equal(g, t)
    dist.barrier()
    # return_size reports what is left behind
    rs = moodist.Queue(pg, location=0, name="sizes")
    if rank == 0:
        for i in range(3):
            rs.put_object(i)
        assert rs.get_object(return_size=True) == (0, 2)
        assert rs.get_tensor(return_size=True)[1] == 1
        assert rs.get_object() == 2
    dist.barrier()
    # many queues at once, spread over the ranks
    many = [moodist.Queue(pg, location=i % world, name=f"many-{i}") for i in range(50)]
    for i, mq in enumerate(many):
        if rank == (i + 1) % world:
            mq.put_object(i)
    for i, mq in enumerate(many):
        if rank == i % world:
            assert mq.get_object(timeout=20) == i
    dist.barrier()
    with pytest.raises(RuntimeError, match="not a rank"):
        moodist.Queue(pg, location=world + 3)
    with pytest.raises(RuntimeError, match="only dense tensors"):
        dq.put_tensor(torch.arange(4).to_sparse())
    if rank == 1:
        dq.put_object(torch.arange(4).to_sparse())  # travels as an object instead
    if rank == 0:
        assert torch.equal(dq.get_object(timeout=20).to_dense(), torch.arange(4))
    # a queue handle dropped while items sit in it leaves the group usable
    doomed = moodist.Queue(pg, location=0, name="doomed")
    if rank == 1:
        for i in range(10):
            doomed.put_object(i)
    dist.barrier()
    del doomed
    gc.collect()
    t = torch.ones(3)
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.barrier()
    dist.destroy_process_group()


def test_queue_edge_cases_world3():
    run_ranks(_edges, 3, timeout=240)


def _producers_and_getters(rank, world, port):
    """Every rank produces 300 items (objects, tensors, transactions of 1-5 items, in random alternation) into a queue
    on rank 0 while rank 0 (locally) and rank 2 (as a remote getter) both consume: nothing is lost, nothing arrives
    twice, and each getter sees each producer's items in the order they were put."""
    import random
    import threading

    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    q = moodist.Queue(pg, location=0, name="many-to-two")
    results = moodist.Queue(pg, location=0, name="what-the-getters-saw")
    count, getters = 300, (0, 2)
    seen, stop = [], threading.Event()

    def consume():
        while not stop.is_set():
            try:
                t = q.get_tensor(timeout=0.2)
            except Empty:
                continue
            seen.append(moodist.deserialize(t) if t.dtype == torch.uint8 else tuple(t.tolist()))

    consumer = None
    if rank in getters:
        consumer = threading.Thread(target=consume)
        consumer.start()
    rng = random.Random(rank)
    i = 0
    while i < count:
        draw = rng.random()
        if draw < 0.3:
            k = min(count - i, rng.randint(1, 5))
            with q.transaction() as tx:
                for j in range(k):
                    tx.put_object((rank, i + j))
            i += k
        elif draw < 0.65:
            q.put_object((rank, i))
            i += 1
        else:
            q.put_tensor(torch.tensor([rank, i]))
            i += 1
    dist.barrier()
    deadline = time.time() + 60
    while rank == 0 and q.qsize() > 0 and time.time() < deadline:
        time.sleep(0.05)
    dist.barrier()
    time.sleep(0.5)  # a getter may hold one more item that was already on its way
    stop.set()
    if consumer is not None:
        consumer.join()
        results.put_object((rank, seen))
    if rank == 0:
        everything = []
        for _ in getters:
            getter, items = results.get_object(timeout=60)
            last = {}
            for producer, number in items:
                assert last.get(producer, -1) < number, (getter, producer, number, last.get(producer))
                last[producer] = number
            everything += items
        assert sorted(everything) == [(p, n) for p in range(world) for n in range(count)], len(everything)
    dist.barrier()
    dist.destroy_process_group()


def test_many_producers_two_getters_exactly_once_in_order():
    run_ranks(_producers_and_getters, 4, timeout=240)


def _multicast_transactions(rank, world, port, seed):
    """Every rank puts single items and transactions of 1-6 items (objects and tensors mixed) into one multicast
    queue that lives on all ranks but the last.  Every location must receive every item, each producer's items
    in the order it put them, and the items of a transaction next to one another although the other ranks put
    at the same time."""
    import random

    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    q = moodist.Queue(pg, location=list(range(world - 1)), name="multicast-transactions")
    rng = random.Random(seed + rank)
    total = 0
    for t in range(60):
        k = rng.randint(1, 6)
        if rng.random() < 0.5:
            with q.transaction() as tx:
                for i in range(k):
                    if rng.random() < 0.5:
                        tx.put_object(("together", rank, t, i, k))
                    else:
                        tx.put_tensor(torch.tensor([rank, t, i, k]))
        else:
            for i in range(k):
                q.put_object(("single", rank, t, i, k))
        total += k
    counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([total]))
    if rank < world - 1:
        items = []
        for _ in range(int(sum(c.item() for c in counts))):
            item = q.get_tensor(timeout=30)
            items.append(moodist.deserialize(item) if item.dtype == torch.uint8 else ("together", *item.tolist()))
        assert q.qsize() == 0
        last = {}
        at = 0
        while at < len(items):
            kind, producer, t, i, k = items[at]
            assert last.get(producer, (-1, -1)) < (t, i), (producer, last.get(producer), t, i)
            if kind == "together":
                assert items[at:at + k] == [("together", producer, t, j, k) for j in range(k)], items[at:at + k]
                at += k
                last[producer] = (t, k - 1)
            else:
                at += 1
                last[producer] = (t, i)
    dist.barrier()
    dist.destroy_process_group()


def test_multicast_queue_keeps_concurrent_transactions_together():
    run_ranks(_multicast_transactions, 4, 5, timeout=240)


def _owner_comes_late(rank, world, port):
    """The producers put (single items, a transaction, more single items) before the owning rank has made its
    first queue: their messages wait on the owner, and must come out in the order in which each producer sent
    them, the transaction's commit between the puts around it."""
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    if rank == 0:
        time.sleep(0.7)
    q = moodist.Queue(pg, location=0, name="late-owner")
    if rank != 0:
        for i in range(20):
            q.put_object((rank, i))
        with q.transaction() as tx:
            for i in range(20, 25):
                tx.put_object((rank, i))
        for i in range(25, 60):
            q.put_object((rank, i))
    else:
        seen = {}
        for _ in range(60 * (world - 1)):
            producer, i = q.get_object(timeout=30)
            assert seen.get(producer, -1) == i - 1, (producer, seen.get(producer), i)
            seen[producer] = i
    dist.barrier()
    dist.destroy_process_group()


def test_messages_that_arrive_before_the_owner_made_its_queue_keep_their_order():
    run_ranks(_owner_comes_late, 3, timeout=120)
