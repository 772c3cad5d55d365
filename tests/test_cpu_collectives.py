"""CPU-tensor collectives over the host engine and TCP transport, world size 2 and 3, checked against a
single-process oracle (the seeded full input is known to every rank)."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _full(world, n, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(world, n, generator=g)
    if dtype in (torch.int32, torch.int64):
        return (x * 100).to(dtype)
    return x.to(dtype)


def _collectives(rank, world, port, n):
    dist = init_moodist(rank, world, port)
    # all_reduce (sum)
    full = _full(world, n, torch.float32)
    t = full[rank].clone()
    dist.all_reduce(t)
    torch.testing.assert_close(t, full.sum(0), rtol=1e-5, atol=1e-5)
    # all_gather_into_tensor
    out = torch.empty(world * n)
    dist.all_gather_into_tensor(out, full[rank].contiguous())
    assert torch.equal(out.view(world, n), full)
    # reduce_scatter_tensor (avg): rank r's input is [world, n]; chunk d goes to rank d
    g = torch.Generator().manual_seed(1)
    allin = torch.randn(world, world, n, generator=g)
    o = torch.empty(n)
    dist.reduce_scatter_tensor(o, allin[rank].reshape(-1).contiguous(), op=dist.ReduceOp.AVG)
    torch.testing.assert_close(o, allin[:, rank].mean(0), rtol=1e-5, atol=1e-6)
    # broadcast from rank 0
    b = full[0].clone() if rank == 0 else torch.zeros(n)
    dist.broadcast(b, src=0)
    assert torch.equal(b, full[0])
    # min / max / int / bf16
    for dtype, op, ref in [
        (torch.int64, dist.ReduceOp.MAX, lambda x: x.max(0).values),
        (torch.int32, dist.ReduceOp.MIN, lambda x: x.min(0).values),
        (torch.float64, dist.ReduceOp.SUM, lambda x: x.sum(0)),
    ]:
        f = _full(world, 257, dtype, seed=3)
        t = f[rank].clone()
        dist.all_reduce(t, op=op)
        assert torch.equal(t, ref(f)), (dtype, op)
    f = _full(world, 1000, torch.bfloat16, seed=4)
    t = f[rank].clone()
    dist.all_reduce(t)
    torch.testing.assert_close(t.float(), f.float().sum(0), rtol=2e-2, atol=2e-2)
    # gather / scatter / all_to_all / barrier
    outs = [torch.empty(5) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.full((5,), float(rank)), outs, dst=0)
    if rank == 0:
        for r in range(world):
            assert bool((outs[r] == r).all())
    s = torch.empty(4)
    dist.scatter(s, [torch.full((4,), float(10 + r)) for r in range(world)] if rank == 0 else None, src=0)
    assert bool((s == 10 + rank).all())
    splits = [[(s_ * 3 + d) % 4 for d in range(world)] for s_ in range(world)]
    inp = torch.cat([torch.full((splits[rank][d], 2), float(rank * 10 + d)) for d in range(world)])
    outp = torch.empty(sum(splits[s_][rank] for s_ in range(world)), 2)
    dist.all_to_all_single(outp, inp, [splits[s_][rank] for s_ in range(world)], splits[rank])
    ref = torch.cat([torch.full((splits[s_][rank], 2), float(s_ * 10 + rank)) for s_ in range(world)])
    assert torch.equal(outp, ref)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 1 << 20), (3, 12345), (1, 100), (8, 4097)])
def test_cpu_collectives(world, n):
    run_ranks(_collectives, world, n, timeout=120)


def _odd_sizes(rank, world, port):
    dist = init_moodist(rank, world, port)
    for n in (1, 2, 3, 7, 9, 64, 255, 1024, 4097):
        full = _full(world, n, torch.float32, seed=n)
        t = full[rank].clone()
        dist.all_reduce(t)
        torch.testing.assert_close(t, full.sum(0), rtol=1e-5, atol=1e-5)
    # above 1 MiB a count that the world does not divide runs as an in-place body plus a round for the remainder
    for n in ((1 << 19) + 1, 3 * (1 << 18) + world - 1):
        full = _full(world, n, torch.float32, seed=n)
        t = full[rank].clone()
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        torch.testing.assert_close(t, full.mean(0), rtol=1e-5, atol=1e-6)
        big = torch.full((n,), rank + 1, dtype=torch.int64)
        dist.all_reduce(big, op=dist.ReduceOp.MAX)
        assert int(big[0]) == world and int(big[-1]) == world
    for i in range(100):  # back to back, mixed
        t = torch.full((16,), float(rank + i))
        dist.all_reduce(t)
        assert bool((t == sum(r + i for r in range(world))).all())
        o = torch.empty(world * 16)
        dist.all_gather_into_tensor(o, t)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_odd_sizes_and_stress(world):
    run_ranks(_odd_sizes, world, timeout=180)


def _send_recv(rank, world, port):
    dist = init_moodist(rank, world, port)
    # a ring of point-to-point messages with tags, two in flight per pair, different sizes
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    a = torch.arange(1000, dtype=torch.float32) + rank
    b = torch.full((3, 7), rank, dtype=torch.int64)
    ra, rb = torch.empty(1000), torch.empty(3, 7, dtype=torch.int64)
    if rank % 2 == 0:
        dist.send(a, nxt, tag=1)
        dist.send(b, nxt, tag=2)
        dist.recv(rb, prv, tag=2)  # received out of send order: matched by tag
        dist.recv(ra, prv, tag=1)
    else:
        dist.recv(rb, prv, tag=2)
        dist.recv(ra, prv, tag=1)
        dist.send(a, nxt, tag=1)
        dist.send(b, nxt, tag=2)
    assert torch.equal(ra, torch.arange(1000, dtype=torch.float32) + prv)
    assert torch.equal(rb, torch.full((3, 7), prv, dtype=torch.int64))
    # non-blocking forms
    reqs = [dist.isend(a * 2, nxt, tag=9), dist.irecv(ra, prv, tag=9)]
    for r in reqs:
        r.wait()
    assert torch.equal(ra, (torch.arange(1000, dtype=torch.float32) + prv) * 2)
    dist.barrier()
    dist.destroy_process_group()


def test_send_recv_ring():
    run_ranks(_send_recv, 2, timeout=120)
    run_ranks(_send_recv, 4, timeout=120)


def _receive_first(rank, world, port):
    dist = init_moodist(rank, world, port)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    # a ring in which every rank posts its receive before its send: irecv must not block
    got, mine = torch.empty(1000), torch.full((1000,), float(rank))
    for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, got, prv), dist.P2POp(dist.isend, mine, nxt)]):
        w.wait()
    assert bool((got == prv).all())
    # two receives from one source with one tag: the order they were posted in decides, not the order of the waits
    if rank == 0:
        dist.send(torch.full((4,), 1.0), 1, tag=5)
        dist.send(torch.full((4,), 2.0), 1, tag=5)
    if rank == 1:
        first, second = torch.empty(4), torch.empty(4)
        w1 = dist.irecv(first, 0, tag=5)
        w2 = dist.irecv(second, 0, tag=5)
        w2.wait()
        w1.wait()
        assert float(first[0]) == 1.0 and float(second[0]) == 2.0 and w1.is_completed()
    # a posted receive whose handle was dropped still has somewhere to put its message
    if rank == 1:
        w = dist.irecv(torch.empty(4), 0, tag=9)
        del w
    dist.barrier()
    if rank == 0:
        dist.send(torch.ones(4), 1, tag=9)
    dist.barrier()
    # a message of another size is an error on the receiver, and the group stays usable
    if rank == 0:
        dist.send(torch.ones(3), 1, tag=11)
    if rank == 1:
        with pytest.raises(RuntimeError, match="size mismatch"):
            dist.recv(torch.empty(5), 0, tag=11)
    # a receive that names no source takes the first message of any rank and says whose it was
    if rank == 0:
        senders = set()
        for _ in range(world - 1):
            box = torch.empty(3)
            who = dist.recv(box, tag=40)
            assert float(box[0]) == who and who not in senders
            senders.add(who)
        assert senders == set(range(1, world))
        big_box = torch.empty(200_000)
        assert dist.recv(big_box, tag=41) == world - 1 and float(big_box[-1]) == 7.0
    else:
        dist.send(torch.full((3,), float(rank)), 0, tag=40)
        if rank == world - 1:
            dist.send(torch.full((200_000,), 7.0), 0, tag=41)
    dist.barrier()
    # large payloads are not copied into a message: the receiver fetches them from the sender's tensor. Sends posted
    # before receives and the other way round, several in flight, then the blocking forms
    n = 300_000
    for sends_first in (True, False):
        outs = [torch.full((n,), float(10 * rank + k)) for k in range(3)]
        ins = [torch.empty(n) for _ in range(3)]
        sends = [dist.P2POp(dist.isend, outs[k], nxt, tag=20 + k) for k in range(3)]
        recvs = [dist.P2POp(dist.irecv, ins[k], prv, tag=20 + k) for k in range(3)]
        for w in dist.batch_isend_irecv(sends + recvs if sends_first else recvs + sends):
            w.wait()
        for k in range(3):
            assert float(ins[k][0]) == 10 * prv + k and float(ins[k][-1]) == 10 * prv + k
    big = torch.arange(n, dtype=torch.float64) + rank
    if rank == 0:
        dist.send(big, 1, tag=30)
    if rank == 1:
        got = torch.empty(n, dtype=torch.float64)
        dist.recv(got, 0, tag=30)
        assert torch.equal(got, torch.arange(n, dtype=torch.float64))
    # a large message of another size fails on both sides, with the reason
    if rank == 0:
        with pytest.raises(RuntimeError, match="size mismatch"):
            dist.send(torch.ones(n), 1, tag=31)
    if rank == 1:
        with pytest.raises(RuntimeError, match="size mismatch"):
            dist.recv(torch.empty(n + 1), 0, tag=31)
    t = torch.ones(2)
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.destroy_process_group()


def test_receives_posted_before_sends():
    run_ranks(_receive_first, 3, timeout=120)


def _many_ranks(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    for n in (1, 1000, 100003):
        x = torch.full((n,), float(rank))
        dist.all_reduce(x)
        assert float(x[0]) == world * (world - 1) / 2 and float(x[-1]) == world * (world - 1) / 2
        out = torch.empty(world * n)
        dist.all_gather_into_tensor(out, torch.full((n,), float(rank)))
        assert float(out[-1]) == world - 1
        o = torch.empty(n)
        dist.reduce_scatter_tensor(o, torch.full((world * n,), 1.0))
        assert float(o[0]) == world
        b = torch.full((n,), float(rank))
        dist.broadcast(b, src=world - 1)
        assert float(b[0]) == world - 1
    send = torch.cat([torch.full((d + 1,), float(rank * 100 + d)) for d in range(world)])
    recv = torch.empty(world * (rank + 1))
    dist.all_to_all_single(recv, send, output_split_sizes=[rank + 1] * world, input_split_sizes=[d + 1 for d in range(world)])
    assert [float(recv[s * (rank + 1)]) for s in range(world)] == [float(s * 100 + rank) for s in range(world)]
    q = moodist.Queue(pg, location=range(world), name="to-everyone")
    if rank == 3:
        q.put_object("hello everyone")
    assert q.get_object(timeout=60) == "hello everyone"
    rows = 4
    op = moodist.compile_op(pg, shape=(rows * world, 8), dtype=torch.float32,
                            inputs=[{"offset": [rank * rows, 0], "shape": [rows, 8]}],
                            outputs=[{"offset": [0, 0], "shape": [rows * world, 8]}])
    out = torch.empty(rows * world, 8)
    op([torch.full((rows, 8), float(rank))], [out]).wait()
    assert out[::rows, 0].tolist() == [float(r) for r in range(world)]
    stats = pg.host_stats()
    assert stats["unix_socket_peers"] == world - 1, stats
    dist.barrier()
    dist.destroy_process_group()


def test_sixteen_cpu_ranks():
    """Twice as many ranks as a node has GPUs: the host engine, the multicast queue and compile_op have no such limit."""
    run_ranks(_many_ranks, 16, timeout=300)


def _mismatch(rank, world, port, kind):
    dist = init_moodist(rank, world, port)
    dist.barrier()
    if kind == "size":
        with pytest.raises(RuntimeError, match="the ranks disagree on sizes"):
            dist.all_reduce(torch.ones(100 if rank == 0 else 200))
    else:
        # whichever check sees it first: the operation codes differ, and so do the sizes the two operations announce
        with pytest.raises(RuntimeError, match="mismatched collectives|the ranks disagree on sizes"):
            if rank == 0:
                dist.all_reduce(torch.ones(100))
            else:
                dist.all_gather_into_tensor(torch.empty(100 * world), torch.ones(100))


@pytest.mark.parametrize("kind", ["size", "operation"])
def test_ranks_that_disagree_get_an_error_not_a_hang(kind):
    run_ranks(_mismatch, 2, kind, timeout=60)


def _random_operations(rank, world, port, seed, count):
    """Every rank draws the same sequence of operations, roots, sizes and peers from one seed and checks every
    result: collectives of all kinds and sizes, point-to-point with either end posted first, a multicast queue,
    a compiled redistribution, back to back in random order."""
    import random

    import moodist_b200 as moodist

    dist = init_moodist(rank, world, port)
    pg = moodist.get_backend(device="cpu")
    q = moodist.Queue(pg, location=range(world), name="random-operations")
    rows = 3
    reshard = moodist.compile_op(pg, shape=(rows * world, 5), dtype=torch.float32,
                                 inputs=[{"offset": [rank * rows, 0], "shape": [rows, 5]}],
                                 outputs=[{"offset": [0, 0], "shape": [rows * world, 5]}])
    rng = random.Random(seed)
    kinds = ["all_reduce", "all_reduce_max", "all_gather", "reduce_scatter", "broadcast", "all_to_all", "p2p", "queue",
             "compile_op", "gather", "barrier"]
    for i in range(count):
        kind = rng.choice(kinds)
        n = rng.choice([1, 7, 100, 4097, 70_001, 300_000])
        where = (i, kind, n)
        if kind == "all_reduce":
            t = torch.full((n,), float(rank + i))
            dist.all_reduce(t)
            assert float(t[-1]) == sum(r + i for r in range(world)), where
        elif kind == "all_reduce_max":
            t = torch.full((n,), rank + i, dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            assert int(t[0]) == world - 1 + i, where
        elif kind == "all_gather":
            out = torch.empty(world * n)
            dist.all_gather_into_tensor(out, torch.full((n,), float(rank * 3 + i)))
            assert [float(out[r * n]) for r in range(world)] == [float(r * 3 + i) for r in range(world)], where
        elif kind == "reduce_scatter":
            out = torch.empty(n)
            dist.reduce_scatter_tensor(out, torch.full((world * n,), float(rank)), op=dist.ReduceOp.AVG)
            assert abs(float(out[0]) - (world - 1) / 2) < 1e-5, where
        elif kind == "broadcast":
            root = rng.randrange(world)
            t = torch.full((n,), float(rank))
            dist.broadcast(t, src=root)
            assert float(t[-1]) == root, where
        elif kind == "all_to_all":
            send = torch.cat([torch.full((d + 1,), float(rank * 100 + d)) for d in range(world)])
            recv = torch.empty(world * (rank + 1))
            dist.all_to_all_single(recv, send, output_split_sizes=[rank + 1] * world, input_split_sizes=[d + 1 for d in range(world)])
            assert float(recv[0]) == rank and float(recv[-1]) == (world - 1) * 100 + rank, where
        elif kind == "p2p":
            shift = rng.randrange(1, world)
            dst, src = (rank + shift) % world, (rank - shift) % world
            got = torch.empty(n)
            ops = [dist.P2POp(dist.isend, torch.full((n,), float(rank + i)), dst, tag=i), dist.P2POp(dist.irecv, got, src, tag=i)]
            for w in dist.batch_isend_irecv(ops if rng.random() < 0.5 else ops[::-1]):
                w.wait()
            assert float(got[-1]) == src + i, where
        elif kind == "queue":
            who = rng.randrange(world)
            if rank == who:
                q.put_object((i, who))
            assert q.get_object(timeout=60) == (i, who), where
        elif kind == "compile_op":
            out = torch.empty(rows * world, 5)
            reshard([torch.full((rows, 5), float(rank + i))], [out]).wait()
            assert out[::rows, 0].tolist() == [float(r + i) for r in range(world)], where
        elif kind == "gather":
            root = rng.randrange(world)
            parts = [torch.empty(3) for _ in range(world)] if rank == root else None
            dist.gather(torch.full((3,), float(rank)), parts, dst=root)
            if rank == root:
                assert [float(x[0]) for x in parts] == [float(r) for r in range(world)], where
        else:
            dist.barrier()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,seed", [(4, 1), (3, 3)])
def test_random_sequences_of_operations(world, seed):
    run_ranks(_random_operations, world, seed, 250, timeout=300)


def _any_dtype(rank, world, port):
    dist = init_moodist(rank, world, port)
    # operations that only move bytes take every dtype, also those that cannot be reduced
    for dtype in (torch.float8_e4m3fn, torch.float8_e5m2, torch.uint16, torch.uint32, torch.complex128, torch.bool):
        mine = (torch.arange(24) % 2 + rank).to(torch.float32).to(dtype)
        first = (torch.arange(24) % 2).to(torch.float32).to(dtype)
        out = torch.zeros(24 * world).to(dtype)
        dist.all_gather_into_tensor(out, mine)
        assert torch.equal(out.view(torch.uint8).view(world, -1)[rank], mine.view(torch.uint8)), dtype
        assert torch.equal(out.view(torch.uint8).view(world, -1)[0], first.view(torch.uint8)), dtype
        got = mine.clone()
        dist.broadcast(got, 0)
        assert torch.equal(got.view(torch.uint8), first.view(torch.uint8)), dtype
        swapped = torch.zeros(24).to(dtype)
        dist.all_to_all_single(swapped, mine)
        if rank == 0:
            dist.send(mine, 1)
        elif rank == 1:
            dist.recv(got, 0)
            assert torch.equal(got.view(torch.uint8), first.view(torch.uint8)), dtype
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        dist.all_reduce(torch.ones(8).to(torch.float8_e4m3fn))
    # views that are not contiguous are refused by name before anything is sent
    grid = torch.zeros(6, 6)
    with pytest.raises(RuntimeError, match="all_reduce tensor must be contiguous"):
        dist.all_reduce(grid.t())
    with pytest.raises(RuntimeError, match="broadcast tensor must be contiguous"):
        dist.broadcast(grid[::2, 1::2], 0)
    if rank == 0:
        with pytest.raises(RuntimeError, match="send tensor must be contiguous"):
            dist.send(grid.t(), 1)
    x = torch.tensor(float(rank))  # no dimensions, and no elements
    dist.all_reduce(x)
    assert x.item() == sum(range(world))
    dist.all_reduce(torch.empty(0))
    dist.barrier()
    dist.destroy_process_group()


def test_moving_operations_take_any_dtype_and_views_are_refused():
    run_ranks(_any_dtype, 3, timeout=120)
