"""Quick correctness check of a process group (CUDA, or CPU ranks on the host path) against a CPU oracle.

``run_selfcheck(group)`` runs every collective the backend serves — all-gather, reduce-scatter (sum and
average), all-reduce, broadcast, uneven all-to-all — at one size per kernel family (small pushes, NVLS
multimem, peer pulls), plus one small all-gather GEMM and one GEMM reduce-scatter, on inputs generated from
per-rank seeds.  Every rank regenerates all ranks' inputs on the CPU, computes the expected result there in
fp32 and compares.  The benchmark runs it before its warm-up whenever more than one GPU takes part, so a
multi-GPU number always comes with evidence that the kernels that produced it compute the right thing.

The reference's tests check collectives the same way (``tests/test_processgroup.py``: results against
values every rank can compute locally).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _data(rank: int, case: int, n: int, dtype) -> torch.Tensor:
    g = torch.Generator().manual_seed(7919 * case + rank)
    x = torch.rand(n, generator=g) * 2 - 1
    return x.to(dtype).float()  # the values the GPU sees, as fp32


class _Checker:
    def __init__(self, group, device):
        self.group, self.device = group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.worst = 0.0
        self.failed = []
        self.cases = 0

    def compare(self, name: str, got: torch.Tensor, want: torch.Tensor, tol: float) -> None:
        got = got.detach().float().cpu().reshape(-1)
        want = want.reshape(-1)
        denom = float(want.abs().max()) + 1e-6
        err = float((got - want).abs().max()) / denom if want.numel() else 0.0
        if not (err == err):  # NaN
            err = float("inf")
        self.worst = max(self.worst, err)
        self.cases += 1
        if err > tol:
            self.failed.append(f"{name}: rel err {err:.3g} > {tol:g}")


def run_selfcheck(group=None, device=None, fused: bool = True) -> dict:
    """Returns ``{"ok", "max_rel_err", "cases", "failed", "variants"}``; a collective, call on every rank."""
    group = group if group is not None else dist.group.WORLD
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    on_gpu = device.type == "cuda"
    ck = _Checker(group, device)
    w, r = ck.world, ck.rank
    backend = None
    if dist.get_backend(group) == "moodist":
        from ..backend import get_backend

        backend = get_backend(group, device=device.type)
    before = backend.stats(False) if backend is not None and on_gpu else {}
    case = 0

    # ---- all-gather: 4 KiB (push), 256 KiB (NVLS where available), 8 MiB (pull) per rank, bf16 ----
    for nbytes in (4 << 10, 256 << 10, 8 << 20):
        case += 1
        n = nbytes // 2
        x = _data(r, case, n, torch.bfloat16).to(device=device, dtype=torch.bfloat16)
        out = torch.empty(w * n, device=device, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(out, x, group=group)
        want = torch.cat([_data(p, case, n, torch.bfloat16) for p in range(w)])
        ck.compare(f"all_gather {nbytes}B", out, want, 0.0)

    # ---- reduce-scatter: fp32 sum and bf16 average, fp32 accumulation ----
    for nbytes, dtype, op in ((4 << 10, torch.float32, dist.ReduceOp.SUM), (256 << 10, torch.bfloat16, dist.ReduceOp.AVG),
                              (4 << 20, torch.float32, dist.ReduceOp.AVG), (4 << 20, torch.bfloat16, dist.ReduceOp.SUM)):
        case += 1
        n = nbytes // (4 if dtype == torch.float32 else 2)
        x = _data(r, case, w * n, dtype).to(device=device, dtype=dtype)
        out = torch.empty(n, device=device, dtype=dtype)
        dist.reduce_scatter_tensor(out, x, op=op, group=group)
        want = sum(_data(p, case, w * n, dtype)[r * n : (r + 1) * n].double() for p in range(w))
        if op == dist.ReduceOp.AVG:
            want = want / w
        ck.compare(f"reduce_scatter {nbytes}B {dtype} {op}", out, want.float(), 1e-5 if dtype == torch.float32 else 1e-2)

    # ---- all-reduce: one-shot, two-shot / NVLS ----
    for nbytes, dtype, op in ((64 << 10, torch.float32, dist.ReduceOp.SUM), (4 << 20, torch.float32, dist.ReduceOp.SUM),
                              (1 << 20, torch.bfloat16, dist.ReduceOp.AVG)):
        case += 1
        n = nbytes // (4 if dtype == torch.float32 else 2)
        x = _data(r, case, n, dtype).to(device=device, dtype=dtype)
        dist.all_reduce(x, op=op, group=group)
        want = sum(_data(p, case, n, dtype).double() for p in range(w))
        if op == dist.ReduceOp.AVG:
            want = want / w
        ck.compare(f"all_reduce {nbytes}B {dtype} {op}", x, want.float(), 1e-5 if dtype == torch.float32 else 1e-2)

    # ---- broadcast from the last rank ----
    case += 1
    n = (1 << 20) // 4
    root = w - 1
    x = _data(r, case, n, torch.float32).to(device)
    dist.broadcast(x, src=dist.get_global_rank(group, root), group=group)
    ck.compare("broadcast 1MiB", x, _data(root, case, n, torch.float32), 0.0)

    # ---- uneven all-to-all: rank s sends (3 s + 5 d + 1) * 1024 elements to rank d ----
    case += 1
    def cnt(s, d):
        return (3 * s + 5 * d + 1) * 1024

    send_counts = [cnt(r, d) for d in range(w)]
    recv_counts = [cnt(s, r) for s in range(w)]
    x = _data(r, case, sum(send_counts), torch.bfloat16).to(device=device, dtype=torch.bfloat16)
    out = torch.empty(sum(recv_counts), device=device, dtype=torch.bfloat16)
    dist.all_to_all_single(out, x, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    parts = []
    for s in range(w):
        full = _data(s, case, sum(cnt(s, d) for d in range(w)), torch.bfloat16)
        off = sum(cnt(s, d) for d in range(r))
        parts.append(full[off : off + cnt(s, r)])
    ck.compare("all_to_all uneven", out, torch.cat(parts), 0.0)

    # ---- fused collective GEMMs (this library's groups only) ----
    if fused and on_gpu and backend is not None and w > 1:
        from ..ops.fused import ag_gemm, gemm_rs

        case += 1
        k, rows, m = 256, 256, 384
        xs = _data(0, case, m * k, torch.bfloat16).view(m, k)  # the activations are the same on every rank
        wshard = _data(r + 1, case, rows * k, torch.bfloat16).view(rows, k)
        y, _ = ag_gemm(backend, wshard.to(device=device, dtype=torch.bfloat16), xs.to(device=device, dtype=torch.bfloat16),
                       gather_weight=True)
        wfull = torch.cat([_data(p + 1, case, rows * k, torch.bfloat16).view(rows, k) for p in range(w)])
        ck.compare("ag_gemm (weights gathered)", y, xs @ wfull.t(), 2e-2)

        case += 1
        mrows, n2, k2 = 128 * w, 512, 256
        a = _data(r, case, mrows * k2, torch.bfloat16).view(mrows, k2)
        b = _data(r + 100, case, n2 * k2, torch.bfloat16).view(n2, k2)
        out = gemm_rs(backend, a.to(device=device, dtype=torch.bfloat16), b.to(device=device, dtype=torch.bfloat16))
        want = torch.zeros(128, n2, dtype=torch.float64)
        for p in range(w):
            ap = _data(p, case, mrows * k2, torch.bfloat16).view(mrows, k2)[r * 128 : (r + 1) * 128]
            bp = _data(p + 100, case, n2 * k2, torch.bfloat16).view(n2, k2)
            # each rank's partial tile crosses NVLink rounded to bf16, the sum over ranks runs in fp32
            want += (ap @ bp.t()).to(torch.bfloat16).double()
        ck.compare("gemm_rs", out, want.float(), 2e-2)

    if on_gpu:
        torch.cuda.synchronize(device)
    variants = []
    if backend is not None and on_gpu:
        after = backend.stats(False)
        for name, row in after.items():
            if row["calls"] > before.get(name, {}).get("calls", 0):
                variants.append(name)
    # every rank must agree that all ranks passed
    flag = torch.tensor([0.0 if not ck.failed else 1.0, ck.worst], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    ok = flag[0].item() == 0.0
    return {"ok": bool(ok), "max_rel_err": float(flag[1].item()), "cases": ck.cases, "failed": ck.failed,
            "variants": sorted(variants)}
