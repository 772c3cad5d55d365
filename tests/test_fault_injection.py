"""Host-side fault injection (nothing here touches a GPU): messages of the engine are duplicated, delayed and
dropped in the middle of collectives; the store loses messages together with their connections.  Duplicates and
delays must be harmless, a lost engine message must surface as an error with its reason on every rank, and
the store must recover by redialling and retransmitting."""

import time

import pytest
import torch

from moodist_b200.utils.testing import free_port, init_moodist, run_ranks


def _collectives_ok(dist, rank, world, rounds):
    for i in range(rounds):
        x = torch.full((1000,), float(rank + i))
        dist.all_reduce(x)
        assert bool((x == sum(range(world)) + i * world).all())
        out = torch.empty(world * 10)
        dist.all_gather_into_tensor(out, torch.full((10,), float(rank)))
        assert torch.equal(out.view(world, 10)[:, 0], torch.arange(world, dtype=torch.float32))
        dist.barrier()


def _duplicates(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200

    pg = moodist_b200.get_backend(device="cpu")
    dist.barrier()
    pg._inject_faults(duplicate_every=2)  # every second message of every rank goes out twice
    _collectives_ok(dist, rank, world, 30)
    q = moodist_b200.Queue(pg, location=0, name="dups")
    for i in range(20):
        q.put_object((rank, i))
    dist.barrier()
    if rank == 0:
        got = sorted(q.get_object(timeout=10) for _ in range(20 * world))
        assert got == sorted((r, i) for r in range(world) for i in range(20))  # nothing delivered twice
        assert q.qsize() == 0
    pg._inject_faults()
    dist.barrier()
    dist.destroy_process_group()


def test_duplicated_messages_are_dropped_by_sequence_number():
    run_ranks(_duplicates, 3, timeout=120)


def _delays(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200

    pg = moodist_b200.get_backend(device="cpu")
    dist.barrier()
    if rank == 1:
        pg._inject_faults(delay_ms=20)  # one slow rank
    t0 = time.time()
    _collectives_ok(dist, rank, world, 10)
    assert time.time() - t0 > 0.2  # the delay was really applied, and everybody waited for the slow rank
    pg._inject_faults()
    dist.barrier()
    dist.destroy_process_group()


def test_delayed_messages_only_slow_things_down():
    run_ranks(_delays, 3, timeout=120)


def _drops(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200

    pg = moodist_b200.get_backend(device="cpu")
    _collectives_ok(dist, rank, world, 3)
    if rank == 1:
        pg._inject_faults(drop_every=5)
    t0 = time.time()
    with pytest.raises(RuntimeError) as info:
        _collectives_ok(dist, rank, world, 50)
    # a gap shows when the next message from that rank arrives (its heartbeat at the latest); the receiver names
    # it and the others learn the reason from its notice
    assert time.time() - t0 < 20
    assert "lost a message from rank 1" in str(info.value), str(info.value)
    # the group stays failed
    with pytest.raises(RuntimeError, match="lost a message"):
        dist.all_reduce(torch.ones(4))


def test_dropped_message_is_detected_and_reported_everywhere():
    statuses = run_ranks(_drops, 3, timeout=120, expect_failure=True, env={"MOODIST_HEARTBEAT_MS": 1000})
    assert statuses == ["ok"] * 3, statuses


def _store_breaks(rank, world, port):
    from datetime import timedelta

    import moodist_b200

    store = moodist_b200.TcpStore("127.0.0.1", port, "faults", world, rank, timedelta(seconds=30))
    store.set(f"hello{rank}", b"x")
    store.wait([f"hello{r}" for r in range(world)])
    store._inject_faults(3)  # every third message is lost with its connection
    for i in range(20):
        store.set(f"k{rank}/{i}", str(i).encode())
    for r in range(world):
        for i in range(20):
            assert store.get(f"k{r}/{i}") == str(i).encode()
    assert store.add("counter", 1) >= 1
    store.wait(["counter"])
    breaks = store._injected_breaks()
    store._inject_faults(0)
    assert breaks >= 10, breaks
    # an add must be applied exactly once although its message may have been retransmitted
    store.set(f"done{rank}", b"1")
    store.wait([f"done{r}" for r in range(world)])
    assert int(store.get("counter")) == world


def test_store_redials_and_retransmits_after_broken_connections():
    run_ranks(_store_breaks, 4, port=free_port(), timeout=120)


def _store_keepalive(rank, world, port):
    from datetime import timedelta

    import moodist_b200

    store = moodist_b200.TcpStore("127.0.0.1", port, "idle", world, rank, timedelta(seconds=20))
    store.set(f"a{rank}", b"1")
    store.wait([f"a{r}" for r in range(world)])
    time.sleep(1.5)  # several keepalive intervals of silence: pings keep the edges, nobody is dropped
    store.set(f"b{rank}", b"2")
    store.wait([f"b{r}" for r in range(world)])
    assert store.get(f"a{(rank + 1) % world}") == b"1"


def test_store_keepalive_over_idle_edges():
    run_ranks(_store_keepalive, 3, port=free_port(), timeout=60, env={"MOODIST_STORE_KEEPALIVE_MS": 200})


def _store_diagnosis(rank, world, port):
    from datetime import timedelta

    import moodist_b200

    store = moodist_b200.TcpStore("127.0.0.1", port, "diag", world, rank, timedelta(seconds=20))
    store.set(f"up{rank}", b"1")
    store.wait([f"up{r}" for r in range(world)])
    if rank == 0:
        # a key nobody sets, owned by a rank that is not a neighbour in the mesh: the timeout message carries
        # the reports of the ranks along the route and of the owner
        hash_ = moodist_b200._core._C.store_string_hash
        far = [r for r in range(1, world) if r not in store.edges()]
        target = next(k for k in (f"never-set-{i}" for i in range(10_000)) if hash_(k) % world in (far or [world - 1]))
        with pytest.raises(RuntimeError) as info:
            store.wait([target], timedelta(seconds=1))
        text = str(info.value)
        assert "timed out" in text and "(owner)" in text and "has not been set" in text, text
        if far:
            assert "forwards to rank" in text, text  # a rank between this one and the owner reported too
    store.set(f"end{rank}", b"1")
    store.wait([f"end{r}" for r in range(world)])


def test_store_timeout_message_carries_reports_from_the_route():
    run_ranks(_store_diagnosis, 6, port=free_port(), timeout=90)
