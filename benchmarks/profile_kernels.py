"""Small single-GPU cases of the hot kernels, for `ncu` captures and quick timing.

    python benchmarks/profile_kernels.py --kernel gemm      # tcgen05 GEMM 8192^3 bf16 (operands exceed L2)
    python benchmarks/profile_kernels.py --kernel ag_gemm   # fused all-gather -> GEMM kernel on a one-rank group
    python benchmarks/profile_kernels.py --kernel gemm_rs   # fused GEMM -> reduce-scatter kernel, one rank
    python benchmarks/profile_kernels.py --kernel copy      # the collective copy/cast loop (world == 1 path)
    python benchmarks/profile_kernels.py --kernel adamw     # flat-shard AdamW, 256 Mi bf16 parameters
    python benchmarks/profile_kernels.py --kernel ce        # cross-entropy forward + backward, [2048, 128256] bf16
    python benchmarks/profile_kernels.py --kernel swiglu    # SwiGLU forward + backward, [8192, 2 x 14336] bf16
    python benchmarks/profile_kernels.py --kernel gemm --variant 1   # the one-SM GEMM instead of the CTA-pair one

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
    ap.add_argument("--kernel", default="gemm", choices=["gemm", "ag_gemm", "gemm_rs", "copy", "adamw", "ce", "swiglu"])
    ap.add_argument("--variant", type=int, default=0, help="GEMM kernel choice: 0 by shape (CTA pairs), 1 one-SM kernel")
    ap.add_argument("--trans-a", action="store_true")
    ap.add_argument("--trans-b", action="store_true")
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
    from moodist_b200._core import _C
    from moodist_b200.ops import train as T

    _C.gemm_variant(args.variant)
    nbytes = 0
    if args.kernel == "gemm":
        ain = a.t().contiguous() if args.trans_a else a
        bin_ = b.t().contiguous() if args.trans_b else b
        fn = lambda: gemm(ain, bin_, trans_a=args.trans_a, trans_b=args.trans_b)  # noqa: E731
        flops = 2.0 * M * N * K
    elif args.kernel == "adamw":
        n = 256 << 20
        p_, g_ = torch.randn(n, device=dev).bfloat16(), torch.randn(n, device=dev).bfloat16()
        m_, v_ = torch.zeros_like(p_), torch.zeros_like(p_)
        fn = lambda: T.adamw_(p_, g_, m_, v_, 1e-4, step=3)  # noqa: E731
        flops, nbytes = 0.0, n * 14  # reads p, g, m, v and writes p, m, v (2 bytes each)
    elif args.kernel == "ce":
        rows, V = 2048, 128256
        logits = torch.randn(rows, V, device=dev).bfloat16()
        tgt = torch.randint(0, V, (rows,), device=dev)
        one = torch.ones(1, device=dev)

        def fn():
            _, lse = _C.cross_entropy_fwd(logits, tgt, -100)
            _C.cross_entropy_bwd_(logits, tgt, lse, one, 1.0 / rows, -100)

        flops, nbytes = 0.0, rows * V * 2 * 3  # forward reads once, backward reads and writes
    elif args.kernel == "swiglu":
        gu = torch.randn(8192, 2 * 14336, device=dev).bfloat16()
        dy = torch.randn(8192, 14336, device=dev).bfloat16()

        def fn():
            _C.swiglu_fwd(gu)
            _C.swiglu_bwd(gu, dy)

        flops, nbytes = 0.0, 8192 * 14336 * 2 * (3 + 5)  # fwd: 2 in 1 out; bwd: 3 in 2 out (per F columns)
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
    elif nbytes:
        print(f"{args.kernel}: {ms:.3f} ms  {nbytes / ms / 1e6:.0f} GB/s (algorithmic read + write bytes)")
    else:
        nbytes = (256 << 20) * 6
        print(f"{args.kernel}: 1 GiB fp32 -> bf16  {ms:.3f} ms  {nbytes / ms / 1e6:.0f} GB/s (read + write)")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
