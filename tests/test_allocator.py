"""CPU and CUDA allocators: sizes, dtypes, ops, transfers, reuse (the reference's tests/test_allocator.py
cases), plus collectives on heap-resident tensors, which peers read in place."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _cpu_allocator(rank, world, port):
    import moodist_b200 as moodist
    from moodist_b200._core import _C

    before = torch.randn(10)
    moodist.enable_cpu_allocator()
    moodist.enable_cpu_allocator()  # idempotent
    for n in (0, 1, 7, 64, 1000, 4096, 1 << 20, (1 << 24) + 3):
        for dtype in (torch.float32, torch.int64, torch.uint8, torch.bfloat16):
            t = torch.ones(n, dtype=dtype)
            assert n == 0 or _C.cpu_allocator_owns(t)
            assert bool((t == 1).all())
    big = torch.zeros(300 << 20, dtype=torch.uint8)  # larger than the largest size class: own mapping
    assert _C.cpu_allocator_owns(big) and int(big[-1]) == 0
    del big
    a, b = torch.randn(256, 256), torch.randn(256, 256)
    torch.testing.assert_close(a @ b, (a.double() @ b.double()).float(), rtol=1e-4, atol=1e-4)
    ptrs = set()
    for _ in range(50):  # blocks are reused
        t = torch.empty(5000)
        ptrs.add(t.data_ptr())
        del t
    assert len(ptrs) <= 2
    assert not _C.cpu_allocator_owns(before)
    assert "class" in moodist.cpu_allocator_debug()
    # the engine works on allocator memory like on any other
    dist = init_moodist(rank, world, port)
    x = torch.full((1000,), 3.0)
    dist.all_reduce(x)
    assert bool((x == 3.0).all())
    dist.destroy_process_group()


def test_cpu_allocator():
    run_ranks(_cpu_allocator, 1, timeout=120)


def _cuda_allocator(rank, world, port):
    import moodist_b200 as moodist

    moodist.enable_cuda_allocator()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    for n in (1, 1000, 1 << 20, (1 << 26) + 5):
        for dtype in (torch.float32, torch.bfloat16, torch.int64):
            t = torch.ones(n, dtype=dtype, device=dev)
            assert bool((t == 1).all())
    a, b = torch.randn(512, 512, device=dev), torch.randn(512, 512, device=dev)
    torch.testing.assert_close((a @ b).cpu(), a.cpu() @ b.cpu(), rtol=1e-3, atol=1e-3)
    h = torch.arange(1000.0)
    assert torch.equal(h.to(dev).cpu(), h)
    ptrs = set()
    for _ in range(20):
        t = torch.empty(1 << 20, device=dev)
        ptrs.add(t.data_ptr())
        del t
    assert len(ptrs) <= 2  # same-stream reuse
    st = moodist.cuda_allocator_stats(rank)
    assert st["heap_mapped_bytes"] > 0 and st["hits"] > 0
    # a block that a side stream still uses is not handed out again: free it while a long kernel of the side
    # stream reads it (record_stream told the allocator), allocate the same size on the main stream at once
    side = torch.cuda.Stream(dev)
    x = torch.full((1 << 22,), 7.0, device=dev)
    x_ptr = x.data_ptr()
    torch.cuda.synchronize()
    big = torch.randn(16384, 16384, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(big)
    torch.matmul(big, big, out=out)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for _ in range(40):  # some tenths of a second of work on the side stream, few launches
            torch.matmul(big, big, out=out)
        y = x * 2
    x.record_stream(side)
    del x
    z = torch.zeros(1 << 22, device=dev)  # same size, main stream, while the side stream still waits
    still_busy = not side.query()
    # (growing the heap for `y` may have synchronised the device; the claim only holds while the side stream runs)
    assert z.data_ptr() != x_ptr or not still_busy
    z.fill_(-1.0)
    torch.cuda.synchronize()
    assert bool((y == 14.0).all())
    assert moodist.cuda_allocator_stats(rank)["cross_stream_frees"] >= 1
    del y, z
    # without record_stream the same sequence reuses the block in stream order (what the cache is for)
    w = torch.empty(1 << 22, device=dev)
    w_ptr = w.data_ptr()
    del w
    assert torch.empty(1 << 22, device=dev).data_ptr() == w_ptr
    # collectives on heap tensors: peers read them in place
    dist = init_moodist(rank, world, port, device="cuda")
    for n in (1000, (1 << 20) + 3):
        g = torch.Generator().manual_seed(n)
        full = torch.randn(world, n, generator=g)
        out = torch.empty(world * n, device=dev)
        dist.all_gather_into_tensor(out, full[rank].to(dev))
        assert torch.equal(out.cpu().view(world, n), full)
        allin = torch.randn(world, world, n, generator=g)
        o = torch.empty(n, device=dev)
        dist.reduce_scatter_tensor(o, allin[rank].reshape(-1).to(dev), op=dist.ReduceOp.AVG)
        torch.testing.assert_close(o.cpu(), allin[:, rank].mean(0), rtol=1e-5, atol=1e-6)
        t = full[rank].to(dev)
        dist.all_reduce(t)
        torch.testing.assert_close(t.cpu(), full.sum(0), rtol=1e-5, atol=1e-5)
        b = torch.full((n,), float(rank), device=dev)
        dist.broadcast(b, src=world - 1)
        assert bool((b == world - 1).all())
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_cuda_allocator_single_gpu():
    run_ranks(_cuda_allocator, 1, timeout=180)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_cuda_allocator_direct_collectives_2gpu():
    run_ranks(_cuda_allocator, 2, timeout=240, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})


def _tracing(rank, world, port):
    import json
    import os
    import tempfile

    os.chdir(tempfile.mkdtemp())
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    t = torch.ones(10)
    dist.all_reduce(t)  # creates the engine
    moodist.enable_profiling(True)
    for _ in range(5):
        dist.all_reduce(t)
    paths = moodist.enable_profiling(False)
    assert len(paths) == 1 and paths[0].startswith("moodist-trace-cpu-") and paths[0].endswith(f"-{rank}.json")
    events = json.load(open(paths[0]))["traceEvents"]
    assert len(events) >= 10 and all(e["ph"] == "X" and e["dur"] >= 0 for e in events)
    assert {e["name"] for e in events} >= {"reduce_scatter", "all_gather"}
    dist.destroy_process_group()


def test_engine_tracing_writes_chrome_trace():
    run_ranks(_tracing, 2, timeout=60)
