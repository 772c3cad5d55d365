"""moodist.TcpStore over loopback with 2-8 CPU ranks: the behaviours of the reference's
tests/test_store.py (set/get, cross-rank visibility, wait, check, overwrite, binary / empty / 1 MiB values,
100 keys, timeout error, graceful three-phase shutdown, clone, multi-key wait, wait timeout, odd keys,
concurrent writers, operations after a peer shut down, unexpected shutdown), plus the mesh/hash facts."""

import time
from datetime import timedelta

import pytest

from moodist_b200.utils.testing import free_port, run_ranks


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
    # joined with a generous limit (the ranks' processes start seconds apart on a busy machine), then shortened
    store = _store(rank, world, port, key="timeout_test", timeout=timedelta(seconds=30))
    store.set_timeout(timedelta(milliseconds=500))
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
    assert time.time() - t0 < 6  # at most 2 s + 1 s + 50 ms of waiting for the others by design


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


_LEAVER = """
import sys, time
from datetime import timedelta
sys.path.insert(0, {root!r})
import moodist_b200
rank, port, marker = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
store = moodist_b200.TcpStore("127.0.0.1", port, "exit-hook", 2, rank, timedelta(seconds=20))
hash_ = moodist_b200._core._C.store_string_hash
key = next(k for k in (f"kept-by-rank-1-{{i}}" for i in range(1000)) if hash_(k) % 2 == 1)
store.set(f"up{{rank}}", b"1")
store.wait(["up0", "up1"])
if rank == 1:
    store.set(key, b"still here")
    cycle = [store]
    cycle.append(cycle)          # nothing destroys the store before the interpreter winds down
    open(marker, "w").close()    # and this process ends right here
else:
    import os
    while not os.path.exists(marker):
        time.sleep(0.01)
    assert store.get(key) == b"still here"
    t0 = time.time()
    try:
        store.wait(["a key nobody sets"])
        print("the wait returned?", flush=True)
    except RuntimeError as e:
        # told by the leaving rank itself, seconds later; a rank that just vanished would leave this wait to its
        # 20 s timeout
        print(f"ended after {{time.time() - t0:.1f}} s: {{e}}", flush=True)
"""


def test_store_left_alive_at_interpreter_exit_still_shuts_down_in_order(tmp_path):
    """A rank ends its process with its store object still referenced (a cycle): between the interpreter's last
    garbage collection and the exit hook the coordinated shutdown still runs, so the other rank's pending wait ends
    within seconds with the name of the rank that left instead of running into its timeout."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "leaver.py"
    script.write_text(_LEAVER.format(root=root))
    port, marker = free_port(), str(tmp_path / "rank1-done")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(port), marker], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in (0, 1)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert procs[0].returncode == 0 and "store was shut down on rank 1" in outs[0], outs
    assert float(outs[0].split("ended after ")[1].split(" s")[0]) < 10, outs
    assert procs[1].returncode == 0, outs


def test_rendezvous_port_in_use_is_reported_at_once():
    import socket

    import moodist_b200 as moodist

    with socket.socket() as holder:
        holder.bind(("127.0.0.1", 0))
        holder.listen(1)
        port = holder.getsockname()[1]
        t0 = time.time()
        with pytest.raises(RuntimeError, match=f"rank 0 cannot listen on port {port}: Address already in use"):
            moodist.TcpStore("127.0.0.1", port, "busy", 2, 0, timedelta(seconds=30))
        assert time.time() - t0 < 5  # not after the 30 s it would take to notice that nobody joins
    with pytest.raises(RuntimeError, match="bad rank"):
        moodist.TcpStore("127.0.0.1", port, "busy", 2, 5, timedelta(seconds=2))


def _random_store_operations(rank, world, port, seed, break_every, steps):
    """Random operations per rank on keys only this rank writes, checked against a dictionary; then a counter
    that everybody adds to.  With `break_every`, every so many messages are lost together with their connection:
    retransmission must apply an add, a compare_set or a delete exactly once."""
    import os
    import random

    import moodist_b200

    store = moodist_b200.TcpStore("127.0.0.1", port, "random", world, rank, timedelta(seconds=60))
    store.set(f"up{rank}", b"1")
    store.wait([f"up{r}" for r in range(world)])
    if break_every:
        store._inject_faults(break_every)
    rng = random.Random(seed * 100 + rank)
    model = {}
    for step in range(steps):
        key = f"rank{rank}/key{rng.randrange(30)}"
        held = model.get(key)
        op = rng.choice(["set", "get", "add", "compare_set", "delete", "check", "append", "multi"])
        if op == "set":
            model[key] = os.urandom(rng.choice([0, 1, 10, 1000, 70000]))
            store.set(key, model[key])
        elif op == "get" and held is not None:
            assert store.get(key) == held, (step, key)
        elif op == "add" and (held is None or held.lstrip(b"-").isdigit()):
            delta = rng.randint(-5, 5)
            expected = int(held or b"0") + delta
            assert store.add(key, delta) == expected, (step, key)
            model[key] = str(expected).encode()
        elif op == "compare_set":
            new = os.urandom(5)
            if held is None or rng.random() < 0.5:  # an absent key matches an empty expectation
                assert store.compare_set(key, held or b"", new) == new, (step, key)
                model[key] = new
            else:
                assert store.compare_set(key, held + b"?", new) == held, (step, key)
        elif op == "delete":
            assert store.delete_key(key) == (held is not None), (step, key)
            model.pop(key, None)
        elif op == "check":
            assert store.check([key]) == (held is not None), (step, key)
        elif op == "append":
            more = os.urandom(3)
            store.append(key, more)
            model[key] = (held or b"") + more
        elif op == "multi":
            keys = [f"rank{rank}/key{rng.randrange(30)}" for _ in range(3)]
            values = [os.urandom(4) for _ in keys]
            store.multi_set(keys, values)
            model.update(zip(keys, values))
            assert store.multi_get(list(model)[:5]) == list(model.values())[:5], step
    for _ in range(50):
        store.add("shared", 1)
    breaks = store._injected_breaks()
    store._inject_faults(0)
    store.set(f"done{rank}", str(len(model)).encode())
    store.wait([f"done{r}" for r in range(world)])
    assert int(store.get("shared")) == 50 * world
    assert store.num_keys() == sum(int(store.get(f"done{r}")) for r in range(world)) + 2 * world + 1
    assert (breaks > 20) == bool(break_every), breaks


@pytest.mark.parametrize("break_every,steps", [(0, 1000), (7, 250)])
def test_random_store_operations_match_a_dictionary(break_every, steps):
    run_ranks(_random_store_operations, 4, 3, break_every, steps, port=free_port(), timeout=180)
