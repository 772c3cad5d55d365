"""Small single-GPU cases of the hot kernels, for `ncu` captures and quick timing.

    python benchmarks/profile_kernels.py --kernel gemm      # tcgen05 GEMM 8192^3 bf16 (operands exceed L2)
    python benchmarks/profile_kernels.py --kernel ag_gemm   # fused all-gather -> GEMM kernel on a one-rank group
    python benchmarks/profile_kernels.py --kernel gemm_rs   # fused GEMM -> reduce-scatter kernel, one rank
    python benchmarks/profile_kernels.py --kernel copy      # the collective copy/cast loop (world == 1 path)

Each case launches the kernel a handful of times and prints its CUDA-event time; under ncu use
`-k regex:<name> -c 1..3`.  The fused kernels run with MOODIST_FORCE_STAGING=1 (set here), which gives a
one-rank group a staging area so that the same kernels that serve 8 GPUs execute on one.
"""

from __future__ import annotations

import argparse
import os
import sys

os.environ.setdefault("MOODIST_FORCE_STAGING", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import moodist_b200  # noqa: E402
from moodist_b200.ops import fused  # noqa: E402
from moodist_b200.ops.gemm import gemm  # noqa: E402
from moodist_b200.utils.testing import free_port  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="gemm", choices=["gemm", "ag_gemm", "gemm_rs", "copy"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dist.init_process_group("moodist", init_method=f"tcp://127.0.0.1:{free_port()}", rank=0, world_size=1)
    pg = moodist_b200.get_backend()
    M, N, K = args.m, args.n, args.k
    a = torch.randn(M, K, device=dev).bfloat16()
    b = torch.randn(N, K, device=dev).bfloat16()
    if args.kernel == "gemm":
        fn = lambda: gemm(a, b)  # noqa: E731
        flops = 2.0 * M * N * K
    elif args.kernel == "ag_gemm":
        fn = lambda: fused.ag_gemm(pg, a, b)  # noqa: E731
        flops = 2.0 * M * N * K
    elif args.kernel == "gemm_rs":
        fn = lambda: fused.gemm_rs(pg, a, b)  # noqa: E731
        flops = 2.0 * M * N * K
    else:
        x = torch.randn(256 << 20, device=dev)  # 1 GiB fp32 -> bf16 cast copy
        out = torch.empty(256 << 20, device=dev, dtype=torch.bfloat16)
        fn = lambda: pg.all_gather_cast(out, x)  # noqa: E731
        flops = 0.0
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    if flops:
        print(f"{args.kernel}: M={M} N={N} K={K}  {ms:.3f} ms  {flops / ms / 1e9:.0f} TFLOP/s")
    else:
        nbytes = (256 << 20) * 6
        print(f"{args.kernel}: 1 GiB fp32 -> bf16  {ms:.3f} ms  {nbytes / ms / 1e6:.0f} GB/s (read + write)")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
