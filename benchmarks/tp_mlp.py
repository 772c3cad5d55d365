"""Tensor/sequence-parallel MLP block (bf16): x [16384, 8192] sharded on sequence, W1 [8192, 28672]
column-sharded, W2 [28672, 8192] row-sharded.

    fused   : ag_gemm (all-gather -> GEMM, SiLU in the epilogue) then gemm_rs (GEMM -> reduce-scatter)
    baseline: NCCL all_gather_into_tensor + torch.matmul + silu + torch.matmul + NCCL reduce_scatter_tensor

Device-timed, max over ranks. Roofline per fused op = max(FLOPs / measured bf16 peak, NVLink bytes / 770 GB/s).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29542 \
        benchmarks/tp_mlp.py
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import moodist_b200  # noqa: E402
from moodist_b200.ops import fused  # noqa: E402


def timed(fn, barrier, warmup, iters, dev):
    for _ in range(warmup):
        fn()
    barrier()
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
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--comm-ctas", type=int, default=0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("moodist", rank=rank, world_size=world)
    pg = moodist_b200.get_backend()
    nccl = dist.new_group(backend="nccl")
    T, H, F = args.tokens, args.hidden, args.ffn
    t, f = T // world, F // world
    torch.manual_seed(rank)
    x = torch.randn(t, H, device=dev).bfloat16()
    w1 = (torch.randn(f, H, device=dev) * 0.02).bfloat16()   # column shard of W1, stored [f, H] (K-major)
    w2 = (torch.randn(H, f, device=dev) * 0.02).bfloat16()   # row shard of W2, stored [H, f] (K-major for x @ W2)

    def fused_block():
        h, _ = fused.ag_gemm(pg, x, w1, epilogue=1, comm_ctas=args.comm_ctas)  # [T, f] = silu(gather(x) @ w1.T)
        return fused.gemm_rs(pg, h, w2)                                         # [t, H]

    xg = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    yo = torch.empty(t, H, device=dev, dtype=torch.bfloat16)

    def nccl_block():
        dist.all_gather_into_tensor(xg, x, group=nccl)
        h = torch.nn.functional.silu(xg @ w1.t())
        y = h @ w2.t()
        dist.reduce_scatter_tensor(yo, y, group=nccl)
        return yo

    def moodist_unfused_block():
        dist.all_gather_into_tensor(xg, x)
        h = torch.nn.functional.silu(xg @ w1.t())
        y = h @ w2.t()
        dist.reduce_scatter_tensor(yo, y)
        return yo

    # correctness first
    a = fused_block().float()
    b = nccl_block().float()
    rel = ((a - b).abs().max() / b.abs().max()).item()
    bar_m = lambda: dist.barrier()  # noqa: E731
    bar_n = lambda: dist.barrier(group=nccl)  # noqa: E731
    res = {"world": world, "tokens": T, "hidden": H, "ffn": F, "max_rel_diff_vs_nccl": rel}
    res["fused_ms"] = timed(fused_block, bar_m, args.warmup, args.iters, dev)
    res["nccl_cublas_ms"] = timed(nccl_block, bar_n, args.warmup, args.iters, dev)
    res["moodist_unfused_ms"] = timed(moodist_unfused_block, bar_m, args.warmup, args.iters, dev)
    res["ag_gemm_ms"] = timed(lambda: fused.ag_gemm(pg, x, w1, epilogue=1, comm_ctas=args.comm_ctas), bar_m, args.warmup, args.iters, dev)
    h, _ = fused.ag_gemm(pg, x, w1, epilogue=1)
    h = h.clone()
    res["gemm_rs_ms"] = timed(lambda: fused.gemm_rs(pg, h, w2), bar_m, args.warmup, args.iters, dev)
    flops_each = 2.0 * T * H * f
    peak = 1374.6e12
    try:
        peak = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))["bf16_tflops_sustained"] * 1e12
    except Exception:
        pass
    link = 770e9
    ag_bytes = (world - 1) * t * H * 2          # what each GPU must receive
    rs_bytes = (world - 1) * t * H * 2          # bf16 partials each GPU must receive
    res["ag_gemm_roofline_ms"] = max(flops_each / peak, ag_bytes / link) * 1e3
    res["gemm_rs_roofline_ms"] = max(flops_each / peak, rs_bytes / link) * 1e3
    res["ag_gemm_frac_of_roofline"] = res["ag_gemm_roofline_ms"] / res["ag_gemm_ms"]
    res["gemm_rs_frac_of_roofline"] = res["gemm_rs_roofline_ms"] / res["gemm_rs_ms"]
    res["speedup_vs_nccl_cublas"] = res["nccl_cublas_ms"] / res["fused_ms"]
    if rank == 0:
        print(json.dumps(res), flush=True)
        if args.out:
            open(args.out, "w").write(json.dumps(res) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
