"""CUDA tensors through Queue and send / recv on 2 GPUs: the sender's host thread never waits for its GPU, the
receiver gets a CUDA tensor whose bytes crossed NVLink, and the order of items is the order of the put calls
whatever mix of CPU and CUDA tensors they carry."""

import time

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

_BUSY = {}


def _keep_gpu_busy(dev, matmuls=50):
    """Queue a few tenths of a second of GPU work on the current stream with few launches (the host must not
    run into the launch queue's depth, which would make it wait for the GPU by itself)."""
    if dev not in _BUSY:
        a = torch.randn(16384, 16384, device=dev, dtype=torch.bfloat16)
        _BUSY[dev] = (a, torch.empty_like(a))
    a, out = _BUSY[dev]
    for _ in range(matmuls):
        torch.matmul(a, a, out=out)  # ~6 ms each


def _queue_cuda(rank, world, port):
    dist = init_moodist(rank, world, port, device="cuda")
    import moodist_b200

    dev = torch.device("cuda", rank)
    pg = moodist_b200.get_backend()
    t = torch.ones(8, device=dev)
    dist.all_reduce(t)  # the group's CUDA side exists from here on: peers' memory is mapped
    torch.cuda.synchronize()
    q = moodist_b200.Queue(pg, location=0, name="cuda-items")
    n = 1 << 20
    if rank == 1:
        q.put_tensor(torch.zeros(n, device=dev)).wait()  # first use sets the hand-over path up
        torch.cuda.synchronize()
        # a long kernel, then the producer of the data, then the put: the put must return long before the GPU
        # gets there, and the receiver must still see the produced values
        x = torch.zeros(n, device=dev)
        ramp = torch.arange(n, device=dev, dtype=torch.float32)  # (allocating inside the timed part could wait for the GPU)
        x.add_(ramp)  # the first launch of a kernel loads its module, which waits for the GPU: do that now
        x.zero_()
        _keep_gpu_busy(dev, 2)  # warm the matmul up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _keep_gpu_busy(dev)
        ta = time.perf_counter()
        x.add_(ramp)
        tb = time.perf_counter()
        w = q.put_tensor(x)
        host_s = time.perf_counter() - t0
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        gpu_s = time.perf_counter() - t1
        # the host was ahead of the GPU the whole time
        assert gpu_s > 0.05 and host_s < gpu_s, (host_s, gpu_s, "busy %.3f add %.3f put %.3f" % (ta - t0, tb - ta, t1 - tb))
        w.wait()
        # FIFO over a mix of CPU and CUDA items, and a transaction that carries CUDA items
        for i in range(10):
            if i % 2:
                q.put_tensor(torch.full((100,), float(i), device=dev))
            else:
                q.put_tensor(torch.full((100,), float(i)))
        with q.transaction() as tx:
            tx.put_tensor(torch.full((50,), 100.0, device=dev))
            tx.put_object({"n": 101})
            tx.put_tensor(torch.full((50,), 102.0, device=dev).bfloat16())
        try:
            with q.transaction() as tx:
                tx.put_tensor(torch.full((50,), -1.0, device=dev))
                raise KeyError("cancel")
        except KeyError:
            pass
        big = torch.arange(40_000_000, device=dev, dtype=torch.int32)  # 160 MB
        q.put_tensor(big)
        q.put_object("end")
    dist.barrier()
    if rank == 0:
        assert bool((q.get_tensor(timeout=60) == 0).all())
        first = q.get_tensor(timeout=60)
        assert first.is_cuda and first.device == dev
        assert torch.equal(first.cpu(), torch.arange(n, dtype=torch.float32))
        for i in range(10):
            item = q.get_tensor(timeout=60)
            assert item.is_cuda == bool(i % 2), (i, item.device)
            assert bool((item == float(i)).all()), i
        a = q.get_tensor(timeout=60)
        b = q.get_object(timeout=60)
        c = q.get_tensor(timeout=60)
        assert a.is_cuda and bool((a == 100.0).all()) and b == {"n": 101}
        assert c.dtype == torch.bfloat16 and bool((c.float() == 102.0).all())
        big = q.get_tensor(timeout=60)
        assert big.is_cuda and big.dtype == torch.int32 and torch.equal(big[::1_000_000].cpu(), torch.arange(0, 40_000_000, 1_000_000, dtype=torch.int32))
        assert int(big[-1]) == 39_999_999
        assert q.get_object(timeout=60) == "end"  # the cancelled transaction left nothing behind
        assert q.qsize() == 0
    torch.cuda.synchronize()
    dist.barrier()
    # a collective after all that: the status word is clean and the sequence numbers still agree
    t = torch.ones(1000, device=dev)
    dist.all_reduce(t)
    assert bool((t == world).all())
    dist.barrier()
    dist.destroy_process_group()


def test_queue_cuda_tensors_stream_ordered():
    run_ranks(_queue_cuda, 2, timeout=240, env={"MOODIST_DEVICE_TIMEOUT_MS": 20000})


def _send_recv_cuda(rank, world, port):
    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    peer = 1 - rank
    t = torch.ones(8, device=dev)
    dist.all_reduce(t)
    torch.cuda.synchronize()
    n = 3_000_001
    want = lambda r, k: torch.arange(n, dtype=torch.float32) * (k + 1) + r  # noqa: E731
    for k in range(4):
        if rank == 0:
            x = torch.zeros(n, device=dev)
            src = want(0, k).to(dev)
            if k == 0:
                x.add_(src)  # first launches load their modules, which waits for the GPU
                x.zero_()
                _keep_gpu_busy(dev, 2)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            _keep_gpu_busy(dev, 20)
            x.add_(src)
            dist.send(x, peer, tag=k)
            host_s = time.perf_counter() - t0
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            gpu_s = time.perf_counter() - t1
            assert k == 0 or host_s < gpu_s, (k, host_s, gpu_s)  # send did not wait for the stream (k = 0 sets up)
            got = torch.empty(n, device=dev)
            dist.recv(got, peer, tag=100 + k)
            assert torch.equal(got.cpu(), want(1, k))
        else:
            got = torch.empty(n, device=dev)
            dist.recv(got, peer, tag=k)
            assert torch.equal(got.cpu(), want(0, k))
            dist.send(want(1, k).to(dev), peer, tag=100 + k)
    # a heap-resident tensor is read in place by the receiver (no staging copy)
    from moodist_b200.allocator import symmetric_pool

    with symmetric_pool():
        h = torch.full((1 << 18,), float(rank + 5), device=dev)
    got = torch.empty(1 << 18, device=dev)
    if rank == 0:
        dist.send(h, peer)
        dist.recv(got, peer)
    else:
        dist.recv(got, peer)
        dist.send(h, peer)
    assert bool((got == float(peer + 5)).all())
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def test_send_recv_cuda_over_nvlink():
    run_ranks(_send_recv_cuda, 2, timeout=240, env={"MOODIST_DEVICE_TIMEOUT_MS": 20000})
