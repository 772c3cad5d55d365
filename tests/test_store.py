"""moodist.TcpStore over loopback with 2-8 CPU ranks: the behaviours of the reference's
tests/test_store.py (set/get, cross-rank visibility, wait, check, overwrite, binary / empty / 1 MiB values,
100 keys, timeout error, graceful three-phase shutdown, clone, multi-key wait, wait timeout, odd keys,
concurrent writers, operations after a peer shut down, unexpected shutdown), plus the mesh/hash facts."""

import time
from datetime import timedelta

import pytest

from moodist_b200.utils.testing import run_ranks


def _store(rank, world, port, key="test", timeout=timedelta(seconds=20)):
    import moodist_b200 as moodist

    return moodist.TcpStore("127.0.0.1", port, key, world, rank, timeout)


def _barrier(store, rank, world, tag):
    store.set(f"__barrier_{tag}_{rank}", b"1")
    store.wait([f"__barrier_{tag}_{r}" for r in range(world)])


def _basic(rank, world, port):
    store = _store(rank, world, port)
    store.set(f"mykey_{rank}", f"value_from_rank_{rank}".encode())
    assert store.get(f"mykey_{rank}") == f"value_from_rank_{rank}".encode()
    _barrier(store, rank, world, "a")
    for r in range(world):  # cross-rank visibility
        assert store.get(f"mykey_{r}") == f"value_from_rank_{r}".encode()
    # wait: rank 0 waits for a key the last rank sets a little later
    if rank == world - 1:
        time.sleep(0.2)
        store.set("late_key", b"late")
    store.wait(["late_key"])
    assert store.get("late_key") == b"late"
    # check
    assert store.check(["late_key", f"mykey_{(rank + 1) % world}"])
    assert not store.check(["late_key", "does_not_exist"])
    # overwrite (one writer), binary, empty, large, many keys
    if rank == 0:
        store.set("ow", b"v1")
        store.set("ow", b"v2")
        store.set("bin", bytes(range(256)))
        store.set("empty", b"")
        store.set("big", b"x" * (1 << 20))
        for i in range(100):
            store.set(f"many_{i}", str(i).encode())
    _barrier(store, rank, world, "b")
    assert store.get("ow") == b"v2"
    assert store.get("bin") == bytes(range(256))
    assert store.get("empty") == b""
    assert store.get("big") == b"x" * (1 << 20)
    for i in range(0, 100, 7):
        assert store.get(f"many_{i}") == str(i).encode()
    # odd keys
    for k in ("", "k" * 10000, "sp ace/sl:ash\n\t\x00é中"):
        store.set(k + str(rank), b"odd")
        assert store.get(k + str(rank)) == b"odd"
    # concurrent writers to one key: the value is one of the candidates
    store.set("contended", f"w{rank}".encode())
    _barrier(store, rank, world, "c")
    assert store.get("contended") in [f"w{r}".encode() for r in range(world)]
    # extensions: add / compare_set / delete / num_keys
    total = store.add("counter", rank + 1)
    assert 1 <= total <= world * (world + 1) // 2
    _barrier(store, rank, world, "d")
    assert store.add("counter", 0) == world * (world + 1) // 2
    if rank == 0:
        assert store.compare_set("cas", b"", b"first") == b"first"
        assert store.compare_set("cas", b"nope", b"second") == b"first"
        assert store.compare_set("cas", b"first", b"second") == b"second"
        assert store.delete_key("cas") and not store.delete_key("cas")
    assert store.num_keys() > 100
    _barrier(store, rank, world, "e")
    del store


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_store_operations(world):
    run_ranks(_basic, world, timeout=90)


def _timeouts(rank, world, port):
    store = _store(rank, world, port, key="timeout_test", timeout=timedelta(milliseconds=500))
    t0 = time.time()
    with pytest.raises(RuntimeError, match="timed out"):
        store.get("this_key_does_not_exist")
    assert 0.4 < time.time() - t0 < 5
    with pytest.raises(RuntimeError, match="timed out"):
        store.wait(["never_set"], timedelta(milliseconds=300))
    if rank == 0:
        store.set("wk1", b"1")
        store.set("wk2", b"2")
    store.wait(["wk1", "wk2"], timedelta(seconds=10))  # multi-key wait
    _barrier(store, rank, world, "t")
    del store


def test_store_timeouts_and_multi_wait():
    run_ranks(_timeouts, 2, timeout=60)


def _graceful(rank, world, port):
    store = _store(rank, world, port, key="shutdown_test", timeout=timedelta(seconds=30))
    store.set(f"key_{rank}", f"value_{rank}".encode())
    _barrier(store, rank, world, "g1")
    for r in range(world):
        assert store.get(f"key_{r}") == f"value_{r}".encode()
    _barrier(store, rank, world, "g2")
    time.sleep(min(0.01 * rank, 0.5))  # staggered destruction must not raise anywhere
    t0 = time.time()
    del store
    assert time.time() - t0 < 3.5


def test_store_graceful_shutdown():
    run_ranks(_graceful, 4, timeout=60)


def _clone(rank, world, port):
    store = _store(rank, world, port, key="clone_test")
    c = store.clone()
    c.set(f"via_clone_{rank}", b"x")
    assert store.get(f"via_clone_{rank}") == b"x"
    del store  # the clone keeps the store alive
    c.set(f"after_{rank}", b"y")
    assert c.get(f"after_{rank}") == b"y"
    _barrier(c, rank, world, "cl")
    del c


def test_store_clone():
    run_ranks(_clone, 2, timeout=60)


def _unexpected(rank, world, port):
    store = _store(rank, world, port, key="unexpected_shutdown_test", timeout=timedelta(seconds=10))
    store.set(f"key_{rank}", b"value")
    _barrier(store, rank, world, "u")
    if rank == 0:
        del store
        time.sleep(3.0)
    else:
        time.sleep(0.1)
        t0 = time.time()
        with pytest.raises(RuntimeError, match="(?i)shut down"):
            store.wait(["key_that_was_never_set"])
        assert time.time() - t0 < 8  # ended by the peer's exit, well before the 10 s timeout
        for op in (lambda: store.set("after_shutdown", b"v"), lambda: store.get("key_0")):
            with pytest.raises(RuntimeError):
                op()
        del store


def test_store_unexpected_shutdown_is_reported():
    run_ranks(_unexpected, 3, timeout=60)


def test_hash_and_mesh_facts():
    from moodist_b200 import _core

    C = _core._C
    # r = 524287; for c: r = r*42643801 + c (mod 2**64); r % 2147483647
    def ref_hash(s):
        r = 524287
        for ch in s.encode():
            r = (r * 42643801 + ch) % (1 << 64)
        return r % 2147483647

    for s in ("", "a", "hello world", "moodist_pg_key", "x" * 100):
        assert C.store_string_hash(s) == ref_hash(s)
    for world in (1, 2, 3, 4, 5, 8, 16, 64, 257):
        mesh = C.store_mesh(world, 12345)
        assert len(mesh) == world
        for r, adj in enumerate(mesh):
            assert len(adj) <= 4 and r not in adj
            for n in adj:
                assert r in mesh[n]  # symmetric
        # connected
        seen, todo = {0}, [0]
        while todo:
            for n in mesh[todo.pop()]:
                if n not in seen:
                    seen.add(n)
                    todo.append(n)
        assert len(seen) == world
        assert C.store_mesh(world, 12345) == mesh  # deterministic


def _rendezvous(rank, world, port):
    import torch
    import torch.distributed as dist

    import moodist_b200  # noqa: F401

    dist.init_process_group("moodist", init_method=f"moodist://127.0.0.1:{port}?rank={rank}&world_size={world}")
    t = torch.ones(4) * (rank + 1)
    dist.all_reduce(t)
    assert bool((t == sum(range(1, world + 1))).all())
    dist.destroy_process_group()


def test_moodist_rendezvous_url():
    run_ranks(_rendezvous, 2, timeout=90)


def _interop(rank, world, port):
    """The store under torch's own machinery, and torch's store under the backend."""
    import torch
    import torch.distributed as dist

    st = _store(rank, world, port, key="interop", timeout=timedelta(seconds=30))
    # the Store base class's derived operations work on top of set / get / add
    st.multi_set([f"m{rank}a", f"m{rank}b"], [b"1", b"2"])
    assert st.multi_get([f"m{rank}a", f"m{rank}b"]) == [b"1", b"2"]
    st.append(f"ap{rank}", b"x")
    st.append(f"ap{rank}", b"y")
    assert st.get(f"ap{rank}") == b"xy"
    ps = dist.PrefixStore("pfx", st)
    ps.set(f"a{rank}", b"1")
    ps.wait([f"a{r}" for r in range(world)])
    assert st.get(f"pfx/a{rank}") == b"1"
    # gloo bootstraps through this store
    dist.init_process_group("gloo", store=dist.PrefixStore("gloo", st), rank=rank, world_size=world)
    t = torch.ones(3)
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.destroy_process_group()
    # the moodist backend through a PrefixStore of it, then through torch's TCPStore
    dist.init_process_group("moodist", store=dist.PrefixStore("moo", st), rank=rank, world_size=world)
    t = torch.ones(3)
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.destroy_process_group()
    ts = dist.TCPStore("127.0.0.1", port + 11, world, rank == 0, timeout=timedelta(seconds=30))
    dist.init_process_group("moodist", store=ts, rank=rank, world_size=world)
    t = torch.ones(3)
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.destroy_process_group()
    _barrier(st, rank, world, "interop-done")


def test_store_under_torch_and_torch_store_under_the_backend():
    run_ranks(_interop, 3, timeout=240)
