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


def _listening_ports():
    """TCP ports this process listens on (from /proc)."""
    inodes = set()
    for fd in os.listdir("/proc/self/fd"):
        try:
            link = os.readlink(f"/proc/self/fd/{fd}")
        except OSError:
            continue
        if link.startswith("socket:["):
            inodes.add(link[8:-1])
    ports = set()
    for table in ("/proc/net/tcp", "/proc/net/tcp6"):
        for line in open(table).read().splitlines()[1:]:
            field = line.split()
            if field[3] == "0A" and field[9] in inodes:  # state LISTEN
                ports.add((table.endswith("6"), int(field[1].rsplit(":", 1)[1], 16)))
    return sorted(ports)


def _strangers(rank, world, port):
    """Whatever arrives on the ports a rank listens on (a port scanner, a stray client, a damaged stream) costs that
    connection only: the engine and the store keep serving the group."""
    import socket
    import struct
    from datetime import timedelta

    import moodist_b200 as moodist

    dist = init_moodist(rank, world, port)
    store = moodist.TcpStore("127.0.0.1", port + 9, "strangers", world, rank, timedelta(seconds=30))
    dist.barrier()
    if rank == 0:
        ports = _listening_ports()
        assert len(ports) >= 3, ports  # the engine's, the store's, the rendezvous port
        frame = 0x40EA69F4
        junk = [b"GET / HTTP/1.1\r\n\r\n", os.urandom(64), os.urandom(100_000),
                struct.pack("<II", frame, 0xFFFFFFFF) + b"x" * 100,   # a frame that claims 4 GiB
                struct.pack("<II", frame, 8) + os.urandom(8),          # a well-formed frame of noise
                struct.pack("<II", frame, 0), struct.pack("<II", frame + 1, 4) + b"abcd", struct.pack("<II", frame, 1 << 30)]
        for v6, p in ports:
            for payload in junk:
                try:
                    with socket.socket(socket.AF_INET6 if v6 else socket.AF_INET) as s:
                        s.settimeout(1)
                        s.connect(("::1" if v6 else "127.0.0.1", p))
                        s.sendall(payload)
                        time.sleep(0.01)
                except OSError:
                    pass
    dist.barrier()
    for _ in range(20):
        t = torch.ones(1000)
        dist.all_reduce(t)
        assert float(t[0]) == world
    store.set(f"after{rank}", b"1")
    store.wait([f"after{r}" for r in range(world)])
    q = moodist.Queue(moodist.get_backend(device="cpu"), 0, name="after-the-noise")
    q.put_object(rank)
    if rank == 0:
        assert sorted(q.get_object(timeout=10) for _ in range(world)) == list(range(world))
    dist.barrier()
    dist.destroy_process_group()


def test_garbage_on_the_listening_ports_is_survived():
    run_ranks(_strangers, 2, timeout=120)
