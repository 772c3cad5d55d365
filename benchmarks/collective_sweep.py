"""Collective bandwidth sweep: all_gather_into_tensor, reduce_scatter_tensor (sum / avg) and all_reduce on
bf16 and fp32 buffers, powers of two from 4 KiB to 1 GiB per rank, moodist kernels vs NCCL on the same
GPUs. Device-timed (CUDA events), max over ranks, 20 warm-up + 100 timed iterations by default.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29540 \
        benchmarks/collective_sweep.py --out sweep8.jsonl

``--impls`` may also name ``moodist_sym``: the same kernels on buffers allocated from the symmetric heap
(``moodist_b200.allocator.symmetric_pool``, what ``enable_cuda_allocator()`` gives every tensor), which peers
read in place instead of through the staging area, and the forced kernel families ``moodist_p2p`` (peer
loads / stores), ``moodist_nvls`` (multimem through NVSwitch) and ``moodist_ce`` (DMA copies between
one-warp flag kernels, no SM time spent on the transfer); ``moodist`` is the library's own choice.

Bus bandwidth follows the usual convention: AG / RS move (n-1)/n of the gathered buffer per GPU, AR twice that.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import moodist_b200  # noqa: E402,F401


def timed(fn, group_barrier, warmup, iters, dev):
    for _ in range(warmup):
        fn()
    group_barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--ops", default="ag,rs_sum,rs_avg,ar")
    ap.add_argument("--impls", default="moodist,nccl")
    ap.add_argument("--out", default="")
    ap.add_argument("--quick", action="store_true", help="fewer iterations above 64 MiB per rank")
    args = ap.parse_args()

    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("moodist", rank=rank, world_size=world)
    groups = {k: dist.group.WORLD for k in ("moodist", "moodist_sym", "moodist_ce", "moodist_p2p", "moodist_nvls")}
    # forced kernel families, for the variant table (moodist_b200.utils.tuning): -1 lets the library choose
    methods = {"moodist_p2p": 0, "moodist_nvls": 1, "moodist_ce": 2}
    backend = moodist_b200.get_backend()
    sym_pool = None
    if "moodist_sym" in args.impls.split(","):
        from moodist_b200.allocator import symmetric_mem_pool

        sym_pool = symmetric_mem_pool()
    if "nccl" in args.impls.split(","):
        groups["nccl"] = dist.new_group(backend="nccl")
    dtypes = {"bf16": torch.bfloat16, "fp32": torch.float32}
    rows = []
    size = args.min_bytes
    sizes = []
    while size <= args.max_bytes:
        sizes.append(size)
        size *= 2
    for dname in args.dtypes.split(","):
        dt = dtypes[dname]
        es = torch.empty(0, dtype=dt).element_size()
        for nbytes in sizes:
            n = nbytes // es
            # --quick cuts the iteration count above 64 MiB per rank (a full-length 1 GiB point takes seconds per
            # implementation); without it every size gets the stated warm-up and timed iterations
            iters = args.iters if (not args.quick or nbytes <= (64 << 20)) else max(10, args.iters // 5)
            warm = args.warmup if (not args.quick or nbytes <= (64 << 20)) else 5
            for impl in args.impls.split(","):
                g = groups[impl]
                if impl.startswith("moodist"):
                    backend._set_option("method", methods.get(impl, -1))
                torch.manual_seed(rank)
                x = (torch.rand(n, device=dev) * 2 - 1).to(dt)
                big = (torch.rand(world * n, device=dev) * 2 - 1).to(dt) if world * nbytes <= (8 << 30) else None
                out_small = torch.empty(n, device=dev, dtype=dt)
                if impl == "moodist_sym":
                    with torch.cuda.use_mem_pool(sym_pool):
                        x, out_small = x.clone(), out_small.clone()
                        big = big.clone() if big is not None else None
                bar = lambda: dist.barrier(group=g)  # noqa: E731
                for op in args.ops.split(","):
                    if big is None:
                        continue
                    if op == "ag":
                        fn = lambda: dist.all_gather_into_tensor(big, x, group=g)  # noqa: E731
                        factor = (world - 1)
                    elif op == "rs_sum":
                        fn = lambda: dist.reduce_scatter_tensor(out_small, big, group=g)  # noqa: E731
                        factor = (world - 1)
                    elif op == "rs_avg":
                        fn = lambda: dist.reduce_scatter_tensor(out_small, big, op=dist.ReduceOp.AVG, group=g)  # noqa: E731
                        factor = (world - 1)
                    else:
                        if world * nbytes > (2 << 30):
                            continue
                        fn = lambda: dist.all_reduce(big, group=g)  # noqa: E731
                        factor = 2 * (world - 1)
                    ms = timed(fn, bar, warm, iters, dev)
                    busbw = factor * nbytes / (ms * 1e-3) / 1e9
                    row = {"op": op, "impl": impl, "dtype": dname, "bytes_per_rank": nbytes, "world": world,
                           "us": ms * 1e3, "busbw_gbs": busbw}
                    rows.append(row)
                    if rank == 0:
                        print(json.dumps(row), flush=True)
                del x, big, out_small
            torch.cuda.empty_cache()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
