"""CUDA collectives on 2, 4 and 8 GPUs (P2P, NVLS and copy-engine kernels over the symmetric heap) against CPU
oracles; every case runs on as many world sizes as the machine has GPUs for."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

WORLDS = [2, 4, 8]


def _need(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


class _Guarded:
    """An output buffer between two guard bands: the output itself is poison-filled before the collective (a
    kernel that skips part of it leaves poison behind), and the bands must be untouched afterwards (a kernel
    that writes outside its output does not get away with it)."""

    GUARD = 256  # elements on each side

    def __init__(self, n, dtype, dev):
        self.poison = 77 if not dtype.is_floating_point else -12345.0
        self.buf = torch.full((n + 2 * self.GUARD,), self.poison, dtype=dtype, device=dev)
        self.out = self.buf[self.GUARD : self.GUARD + n]
        self.n = n

    def check(self, what):
        torch.cuda.synchronize()
        lo, hi = self.buf[: self.GUARD], self.buf[self.GUARD + self.n :]
        assert bool((lo == self.poison).all()) and bool((hi == self.poison).all()), ("guard band overwritten", what)


def _cuda_collectives(rank, world, port):
    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        for n in (1, 7, 1000, 65536, (1 << 20) + 3):
            g = torch.Generator().manual_seed(n)
            full = (torch.randn(world, n, generator=g) * 10).to(dtype)
            gd = _Guarded(world * n, dtype, dev)
            out = gd.out
            dist.all_gather_into_tensor(out, full[rank].to(dev).contiguous())
            assert torch.equal(out.cpu().view(world, n), full), ("all_gather", dtype, n)
            gd.check(("all_gather", dtype, n))
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2), (torch.int32, 0)):
        for op in (dist.ReduceOp.SUM, dist.ReduceOp.AVG, dist.ReduceOp.MAX, dist.ReduceOp.MIN):
            if dtype == torch.int32 and op == dist.ReduceOp.AVG:
                continue
            for n in (1, 9, 4096, (1 << 18) + 5):
                g = torch.Generator().manual_seed(n)
                allin = (torch.randn(world, world, n, generator=g) * 4).to(dtype)
                gd = _Guarded(n, dtype, dev)
                out = gd.out
                dist.reduce_scatter_tensor(out, allin[rank].reshape(-1).to(dev).contiguous(), op=op)
                gd.check(("reduce_scatter", dtype, op, n))
                col = allin[:, rank].double()
                ref = {dist.ReduceOp.SUM: col.sum(0), dist.ReduceOp.AVG: col.mean(0), dist.ReduceOp.MAX: col.max(0).values,
                       dist.ReduceOp.MIN: col.min(0).values}[op]
                err = (out.double().cpu() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
                assert err <= tol, ("reduce_scatter", dtype, op, n, err)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        for n in (1, 5, 1000, 70000, (1 << 20) + 11):  # one-shot and two-shot paths
            g = torch.Generator().manual_seed(n)
            allin = torch.randn(world, n, generator=g).to(dtype)
            gd = _Guarded(n, dtype, dev)
            t = gd.out
            t.copy_(allin[rank])
            dist.all_reduce(t)
            ref = allin.double().sum(0)
            err = (t.double().cpu() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
            assert err <= tol, ("all_reduce", dtype, n, err)
            gd.check(("all_reduce", dtype, n))
    for root in (0, world - 1):
        t = torch.full((100001,), float(rank + 1), device=dev)
        dist.broadcast(t, src=root)
        assert bool((t == root + 1).all())
    torch.manual_seed(1234)
    splits = torch.randint(0, 50, (world, world))
    H = 64
    inp = torch.cat([torch.full((int(splits[rank, d]), H), rank * 100 + d, dtype=torch.bfloat16) for d in range(world)]).to(dev)
    out = torch.empty(int(splits[:, rank].sum()), H, dtype=torch.bfloat16, device=dev)
    dist.all_to_all_single(out, inp, [int(x) for x in splits[:, rank]], [int(x) for x in splits[rank]])
    ref = torch.cat([torch.full((int(splits[s, rank]), H), s * 100 + rank, dtype=torch.bfloat16) for s in range(world)])
    assert torch.equal(out.cpu(), ref)
    # very uneven splits (the ranks end up with different grid sizes, segments above the two-half threshold
    # next to empty ones), the output once in ordinary memory and once in the symmetric heap
    from moodist_b200.allocator import symmetric_mem_pool

    pool = symmetric_mem_pool()
    for it, rows in enumerate([[0, 3, 40000, 1], [70000, 0, 5, 12345], [17, 17, 17, 17]]):
        sp = torch.zeros(world, world, dtype=torch.long)
        for s_ in range(world):
            for d in range(world):
                sp[s_, d] = rows[(s_ * world + d + it) % len(rows)]
        inp = torch.cat([torch.full((int(sp[rank, d]), H), rank * 10 + d, dtype=torch.bfloat16) for d in range(world)]).to(dev)
        ref = torch.cat([torch.full((int(sp[s_, rank]), H), s_ * 10 + rank, dtype=torch.bfloat16) for s_ in range(world)])
        for symmetric in (False, True):
            if symmetric:
                with torch.cuda.use_mem_pool(pool):
                    out = torch.zeros(int(sp[:, rank].sum()), H, dtype=torch.bfloat16, device=dev)
            else:
                out = torch.zeros(int(sp[:, rank].sum()), H, dtype=torch.bfloat16, device=dev)
            dist.all_to_all_single(out, inp, [int(x) for x in sp[:, rank]], [int(x) for x in sp[rank]])
            assert torch.equal(out.cpu(), ref), ("uneven all_to_all", it, symmetric)
    dist.barrier()
    import moodist_b200

    assert moodist_b200.get_backend().kernel_launches() > 0
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_cuda_collectives(world):
    _need(world)
    run_ranks(_cuda_collectives, world, timeout=300, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})


def _nvls_variants(rank, world, port):
    dist = init_moodist(rank, world, port, device="cuda")
    import moodist_b200

    dev = torch.device("cuda", rank)
    pg = moodist_b200.get_backend()
    t = torch.ones(8, device=dev)
    dist.all_reduce(t)  # creates the CUDA group
    if "nvls=1" not in pg.describe():
        dist.destroy_process_group()
        return  # no multicast support on this machine: nothing to check
    with pg.options(method=1):
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
            for n in (64, 1000, 4096, (1 << 20) + 24):
                g = torch.Generator().manual_seed(n)
                allin = torch.randn(world, n, generator=g).to(dtype)
                x = allin[rank].to(dev).contiguous()
                dist.all_reduce(x)
                ref = allin.double().sum(0)
                err = (x.double().cpu() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
                assert err <= tol, ("nvls all_reduce", dtype, n, err)
                m = (n // 8) * 8
                rs_in = torch.randn(world, world, m, generator=g).to(dtype)
                out = torch.empty(m, device=dev, dtype=dtype)
                dist.reduce_scatter_tensor(out, rs_in[rank].reshape(-1).to(dev).contiguous(), op=dist.ReduceOp.AVG)
                ref = rs_in[:, rank].double().mean(0)
                err = (out.double().cpu() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
                assert err <= tol, ("nvls reduce_scatter", dtype, m, err)
                full = torch.randn(world, n, generator=g).to(dtype)
                ag = torch.empty(world * n, device=dev, dtype=dtype)
                dist.all_gather_into_tensor(ag, full[rank].to(dev).contiguous())
                assert torch.equal(ag.cpu().view(world, n), full), ("nvls all_gather", dtype, n)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_nvls_variants(world):
    _need(world)
    run_ranks(_nvls_variants, world, timeout=300, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})


def _mixed_modes(rank, world, port):
    """Ranks that differ in per-rank facts — only rank 0's tensors live in the symmetric heap, only the last
    rank's pointers are off a 16-byte boundary — still pick the same kernel family and piece count for one
    collective, at sizes of every family (push, NVLS, pull)."""
    dist = init_moodist(rank, world, port, device="cuda")
    import moodist_b200
    from moodist_b200.allocator import symmetric_mem_pool

    dev = torch.device("cuda", rank)
    pool = symmetric_mem_pool()

    def alloc(n, dtype, heap):
        if heap:
            with torch.cuda.use_mem_pool(pool):
                return torch.zeros(n, dtype=dtype, device=dev)
        return torch.zeros(n, dtype=dtype, device=dev)

    for nbytes in (16 << 10, 1 << 20, 8 << 20):
        n = nbytes // 2
        g = torch.Generator().manual_seed(nbytes)
        full = (torch.rand(world, n, generator=g) * 2 - 1).to(torch.bfloat16)
        x = alloc(n, torch.bfloat16, heap=(rank == 0))
        x.copy_(full[rank])
        out = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(out, x)
        assert torch.equal(out.cpu().view(world, n), full), ("mixed all_gather", nbytes)
        # reduce-scatter: rank 0's input in the heap (read in place by the peers), the others staged
        allin = (torch.rand(world, world, n // 4, generator=g) * 2 - 1).to(torch.bfloat16)
        xin = alloc(world * (n // 4), torch.bfloat16, heap=(rank == 0))
        xin.copy_(allin[rank].reshape(-1))
        o = torch.empty(n // 4, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o, xin, op=dist.ReduceOp.AVG)
        torch.testing.assert_close(o.float().cpu(), allin[:, rank].float().mean(0), rtol=2e-2, atol=2e-2)
    # all-reduce in the NVLS size range with one rank's buffer off a 16-byte boundary
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        n = (4 << 20) // (4 if dtype == torch.float32 else 2)
        g = torch.Generator().manual_seed(n)
        allin = torch.randn(world, n, generator=g).to(dtype)
        buf = torch.empty(n + 8, device=dev, dtype=dtype)
        t = buf[1 : n + 1] if rank == world - 1 else buf[:n]
        t.copy_(allin[rank])
        dist.all_reduce(t)
        ref = allin.double().sum(0)
        err = (t.double().cpu() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        assert err <= tol, ("misaligned all_reduce", dtype, err)
    pg = moodist_b200.get_backend()
    if "nvls=1" in pg.describe():
        with pg.options(method=1):  # NVLS reduce-scatter with the output of one rank misaligned
            n = 1 << 18
            g = torch.Generator().manual_seed(3)
            allin = (torch.rand(world, world, n, generator=g) * 2 - 1).to(torch.bfloat16)
            buf = torch.empty(n + 8, device=dev, dtype=torch.float32)
            o = buf[1 : n + 1] if rank == world - 1 else buf[:n]
            pg.reduce_scatter_cast(o, allin[rank].reshape(-1).to(dev), int(dist.ReduceOp.SUM), 1.0)
            # the switch accumulates in fp32 but hands back bf16 values: bf16-sized tolerance
            torch.testing.assert_close(o.cpu(), allin[:, rank].float().sum(0), rtol=2e-2, atol=2e-2)
    stats = pg.stats()
    assert any(k.startswith("all_gather/") for k in stats) and all(v["calls"] > 0 for v in stats.values()), stats
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 8])
def test_mixed_heap_and_alignment_modes(world):
    _need(world)
    run_ranks(_mixed_modes, world, timeout=300, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})


def _stress(rank, world, port):
    """100 back-to-back collectives of each kind and an interleaved mix, small sizes: sequence parity, the two
    staging halves and the per-grid counters are reused hundreds of times (modelled on the reference's
    tests/test_stress.py)."""
    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    sizes = [1, 7, 64, 255, 1024, 4096, 65536]
    for n in sizes:
        x = torch.full((n,), float(rank + 1), device=dev)
        out = torch.empty(world * n, device=dev)
        for _ in range(100):
            dist.all_gather_into_tensor(out, x)
        assert torch.equal(out.view(world, n)[:, 0].cpu(), torch.arange(1, world + 1, dtype=torch.float32)), ("ag", n)
        xin = torch.arange(world * n, device=dev, dtype=torch.float32) + rank
        o = torch.empty(n, device=dev)
        for _ in range(100):
            dist.reduce_scatter_tensor(o, xin)
        want = world * torch.arange(rank * n, (rank + 1) * n, dtype=torch.float32) + sum(range(world))
        assert torch.equal(o.cpu(), want), ("rs", n)
        t = torch.full((n,), 1.0, device=dev)
        for i in range(100):
            t.fill_(float(rank + i))
            dist.all_reduce(t)
        assert bool((t == sum(range(world)) + 99 * world).all()), ("ar", n)
        for i in range(100):
            b = torch.full((n,), float(rank * 1000 + i), device=dev)
            dist.broadcast(b, src=i % world)
            if i == 99:
                assert bool((b == (99 % world) * 1000 + 99).all()), ("bc", n)
    # interleaved mix with a barrier now and then
    for i in range(100):
        n = sizes[i % len(sizes)]
        x = torch.full((n,), float(rank + i), device=dev)
        out = torch.empty(world * n, device=dev)
        dist.all_gather_into_tensor(out, x)
        o = torch.empty(n, device=dev)
        dist.reduce_scatter_tensor(o, out)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        dist.broadcast(o, src=(i + 1) % world)
        if i % 10 == 9:
            dist.barrier()
        assert bool((x == world - 1 + i).all()), ("mix", i)
    for _ in range(10):
        big = torch.full((1 << 20,), float(rank), device=dev)  # 4 MiB
        dist.all_reduce(big)
    assert bool((big == sum(range(world))).all())
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("kernel_less", [False, True])
def test_stress_back_to_back(world, kernel_less):
    _need(world)
    env = {"MOODIST_DEVICE_TIMEOUT_MS": 5000}
    if kernel_less:
        env["MOODIST_CE_MIN_BYTES"] = 0  # every all-gather / reduce-scatter goes through the DMA variant
    run_ranks(_stress_kl if kernel_less else _stress, world, timeout=600, env=env)


def _stress_kl(rank, world, port):
    import moodist_b200

    moodist_b200.set_prefer_kernel_less(True)
    _stress(rank, world, port)


def _copy_engine_variants(rank, world, port):
    """The copy-engine variants (DMA copies between one-warp flag kernels) against the seeded oracle, mixed
    with kernel collectives so that sequence numbers and staging halves interleave."""
    dist = init_moodist(rank, world, port, device="cuda")
    import moodist_b200

    dev = torch.device("cuda", rank)
    pg = moodist_b200.get_backend()
    for it, (dtype, n) in enumerate([(torch.bfloat16, 1 << 20), (torch.float32, 300_000), (torch.bfloat16, 1 << 23),
                                     (torch.float16, 65536 + 8)]):
        pg.set_prefer_kernel_less(it % 2 == 0)
        pg._set_option("method", 2 if it % 2 else -1)  # odd rounds force the copy engine through `method`
        g = torch.Generator().manual_seed(77 + it)
        full = (torch.rand(world, n, generator=g) * 2 - 1).to(dtype)
        ag = torch.empty(world * n, device=dev, dtype=dtype)
        dist.all_gather_into_tensor(ag, full[rank].to(dev).contiguous())
        assert torch.equal(ag.cpu().view(world, n), full), ("ce all_gather", dtype, n)
        # in place: the input is the rank's slice of the output
        ag2 = torch.zeros(world * n, device=dev, dtype=dtype)
        ag2.view(world, n)[rank].copy_(full[rank])
        dist.all_gather_into_tensor(ag2, ag2.view(world, n)[rank])
        assert torch.equal(ag2.cpu().view(world, n), full), ("ce all_gather in place", dtype, n)
        allin = (torch.rand(world, world, n, generator=g) * 2 - 1).to(dtype)
        out = torch.empty(n, device=dev, dtype=dtype)
        dist.reduce_scatter_tensor(out, allin[rank].reshape(-1).to(dev), op=dist.ReduceOp.AVG)
        ref = allin[:, rank].float().mean(0)
        torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-2, atol=2e-2)
        if dtype == torch.bfloat16:
            out32 = torch.empty(n, device=dev, dtype=torch.float32)
            pg.reduce_scatter_cast(out32, allin[rank].reshape(-1).to(dev), int(dist.ReduceOp.SUM), 1.0)
            torch.testing.assert_close(out32.cpu(), allin[:, rank].float().sum(0), rtol=1e-5, atol=1e-5)
        pg._set_option("method", -1)
        pg.set_prefer_kernel_less(False)
        t = torch.ones(4096, device=dev)
        dist.all_reduce(t)  # a kernel collective in between
        assert bool((t == world).all())
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def _composed_all_reduce(rank, world, port):
    """MOODIST_AR_COMPOSE_BYTES: all-reduce as reduce-scatter kernel + in-place all-gather, in and out of place."""
    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    for dtype, n, op in [(torch.bfloat16, 1 << 20, dist.ReduceOp.SUM), (torch.float32, 3 << 19, dist.ReduceOp.AVG),
                         (torch.bfloat16, 64 << 20, dist.ReduceOp.SUM), (torch.float32, 1000, dist.ReduceOp.SUM)]:
        g = torch.Generator().manual_seed(5)
        full = (torch.rand(world, n, generator=g) * 2 - 1).to(dtype)
        t = full[rank].to(dev)
        dist.all_reduce(t, op=op)
        ref = full.float().sum(0) / (world if op == dist.ReduceOp.AVG else 1)
        torch.testing.assert_close(t.float().cpu(), ref, rtol=2e-2, atol=2e-2)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def test_composed_all_reduce_2gpu():
    run_ranks(_composed_all_reduce, 2, timeout=240, env={"MOODIST_AR_COMPOSE_BYTES": 1 << 20,
                                                         "MOODIST_DEVICE_TIMEOUT_MS": 5000})


def test_copy_engine_variants_2gpu():
    run_ranks(_copy_engine_variants, 2, timeout=240, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})


def _cuda_send_recv(rank, world, port):
    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    peer = 1 - rank
    a = (torch.arange(100_000, device=dev, dtype=torch.float32) + rank).bfloat16()
    got = torch.empty_like(a)
    if rank == 0:
        dist.send(a, peer, tag=3)
        dist.recv(got, peer, tag=4)
    else:
        dist.recv(got, peer, tag=3)
        dist.send(a, peer, tag=4)
    want = (torch.arange(100_000, device=dev, dtype=torch.float32) + peer).bfloat16()
    assert torch.equal(got, want)
    dist.barrier()
    dist.destroy_process_group()


def test_cuda_send_recv_2gpu():
    run_ranks(_cuda_send_recv, 2, timeout=120)


def _absent_rank(rank, world, port):
    """A device wait that runs out returns a status instead of hanging: rank 1 never launches."""
    import time

    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    t = torch.ones(1024, device=dev)
    dist.all_reduce(t)
    torch.cuda.synchronize()
    store = dist.distributed_c10d._get_default_store()
    if rank == 0:
        x = torch.ones(1 << 16, device=dev)
        t0 = time.time()
        dist.all_reduce(x)  # the peer is not there: the kernel gives up after the cap
        torch.cuda.synchronize()
        assert time.time() - t0 < 10
        with pytest.raises(RuntimeError, match="timed out"):
            dist.all_reduce(x)
        y = torch.ones(4, device=dev) * 3  # the context is still usable
        assert float(y.sum()) == 12.0
        store.set("rank0_done", b"1")
        store.wait(["rank1_done"])  # rank 0 hosts the store: it leaves last
    else:
        store.wait(["rank0_done"])  # leaves only between steps, nothing of its own in flight
        store.set("rank1_done", b"1")
    import os

    os._exit(0)


def test_absent_rank_times_out_without_hanging():
    statuses = run_ranks(_absent_rank, 2, timeout=120, expect_failure=True,
                         env={"MOODIST_DEVICE_TIMEOUT_MS": 800, "MOODIST_DISABLE_NVLS": 1, "NCCL_NVLS_ENABLE": 0})
    # ranks leave through os._exit(0) without writing a status file; a Python failure would have written one
    for s in statuses:
        assert s.startswith("died with exit code 0"), s
