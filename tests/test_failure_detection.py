"""Failure detection on the host path (CPU ranks, nothing on a GPU): a rank that leaves between steps makes the
others' next collective raise with the reason instead of hanging; a silent peer is reported by the heartbeat."""

import os
import signal
import time

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _rank_leaves(rank, world, port):
    dist = init_moodist(rank, world, port)
    t = torch.ones(1000)
    dist.all_reduce(t)
    assert bool((t == world).all())
    dist.barrier()
    if rank == world - 1:
        # leaves between steps with nothing of its own in flight, without the coordinated shutdown
        os._exit(0)
    time.sleep(0.5)
    t0 = time.time()
    with pytest.raises(RuntimeError) as info:
        for _ in range(50):  # the first call may still complete locally; one of the next ones must fail
            dist.all_reduce(torch.ones(1 << 16))
    assert time.time() - t0 < 30, "the failure took too long to surface"
    text = str(info.value)
    assert "rank" in text or "connection" in text or "error state" in text, text
    # the group stays in its error state: later calls fail at once, with the same reason
    t1 = time.time()
    with pytest.raises(RuntimeError):
        dist.all_reduce(torch.ones(4))
    assert time.time() - t1 < 5
    # returning lets the runner record "ok" and leave without the coordinated shutdown (the peer is gone)


def test_rank_leaving_is_reported_to_the_others():
    statuses = run_ranks(_rank_leaves, 3, timeout=120, expect_failure=True)
    assert statuses[0] == "ok" and statuses[1] == "ok", statuses
    assert "exit code 0" in statuses[2], statuses


def _silent_peer(rank, world, port):
    import signal

    dist = init_moodist(rank, world, port)
    pids = torch.zeros(world, dtype=torch.int64)
    dist.all_gather_into_tensor(pids, torch.tensor([os.getpid()]))
    dist.barrier()
    if rank == 1:
        # stays alive (sockets open) but stops taking part, engine thread included: only the heartbeat can tell
        os.kill(os.getpid(), signal.SIGSTOP)
        return
    t0 = time.time()
    try:
        with pytest.raises(RuntimeError, match="heartbeat|error state|timed out"):
            for _ in range(400):
                dist.all_reduce(torch.ones(16))
                time.sleep(0.05)
        assert time.time() - t0 < 40
    finally:
        os.kill(int(pids[1]), signal.SIGKILL)  # the exact process this test started as rank 1


def test_silent_peer_is_reported_by_the_heartbeat():
    statuses = run_ranks(_silent_peer, 2, timeout=90, expect_failure=True, env={"MOODIST_HEARTBEAT_MS": 500})
    assert statuses[0] == "ok", statuses


def _interrupts(rank, world, port):
    """A signal handler that raises (Ctrl-C) ends a wait that would never end by itself: a get on an empty queue, a
    store wait for a key nobody sets, a receive nobody sends to."""
    import threading
    from datetime import timedelta

    import moodist_b200 as moodist

    dist = init_moodist(rank, world, port)
    pg = moodist.get_backend(device="cpu")
    store = moodist.TcpStore("127.0.0.1", port + 5, "signals", world, rank, timedelta(seconds=60))
    q = moodist.Queue(pg, location=0, name="signals")
    dist.barrier()

    def interrupted(blocking_call):
        threading.Timer(0.5, lambda: signal.raise_signal(signal.SIGINT)).start()
        t0 = time.time()
        with pytest.raises(KeyboardInterrupt):
            blocking_call()
        assert time.time() - t0 < 10

    if rank == 0:
        interrupted(lambda: q.get_object())
        interrupted(lambda: store.wait(["a key nobody sets"]))
        q.put_object("later")  # the queue and the store are as usable as before
        assert q.get_object(timeout=10) == "later"
        store.set("still", b"works")
        assert store.get("still") == b"works"
        # a collective or a receive refers to the caller's buffers: after the interrupt nothing of the group may touch
        # them any more, so the group goes into its error state and tells the others why
        interrupted(lambda: dist.recv(torch.empty(4), src=1))
        with pytest.raises(RuntimeError, match="interrupted by a signal"):
            dist.all_reduce(torch.ones(2))
    else:
        with pytest.raises(RuntimeError, match="rank 0 reported: interrupted by a signal"):
            for _ in range(100):
                dist.all_reduce(torch.ones(2))
                time.sleep(0.1)


def test_a_signal_ends_waits_that_would_never_end():
    run_ranks(_interrupts, 2, timeout=90)
