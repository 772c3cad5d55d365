"""MoE dispatch / combine with uneven all_to_all_single, and a 2-D-block -> 1-D-row compile_op reshard.

64 experts (8 per GPU at 8 GPUs), top-2 routing, 32768 tokens per GPU, hidden 4096 bf16, router logits
N(0,1) from a per-rank seed; per-rank split sizes come from the routing. moodist kernels vs NCCL
all_to_all_single. Reshard: [65536, 8192] bf16 from a (2 x world/2) block layout to row sharding, compile_op vs
NCCL all_gather + slice. Device-timed, max over ranks.
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
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--reshard-rows", type=int, default=65536)
    ap.add_argument("--reshard-cols", type=int, default=8192)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    # the dispatch buffer (tokens x topk x hidden) is 512 MiB per rank: give the staging halves room for it
    os.environ.setdefault("MOODIST_STAGING_MB", "2048")
    dist.init_process_group("moodist", rank=rank, world_size=world)
    nccl = dist.new_group(backend="nccl")
    pg = moodist_b200.get_backend()
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    per_gpu = E // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    logits = torch.randn(T, E, device=dev, generator=g)
    top = logits.topk(K, dim=-1).indices.reshape(-1)          # [T*K] expert ids
    order = torch.argsort(top, stable=True)                    # group token copies by expert (hence by destination rank)
    dest_rank = (top[order] // per_gpu)
    send_counts = torch.bincount(dest_rank, minlength=world)
    # everyone learns everyone's counts
    all_counts = torch.empty(world * world, dtype=send_counts.dtype, device=dev)
    dist.all_gather_into_tensor(all_counts, send_counts)
    all_counts = all_counts.view(world, world).cpu()
    in_split = [int(v) for v in all_counts[rank]]
    out_split = [int(v) for v in all_counts[:, rank]]
    x = torch.randn(T, H, device=dev, generator=g).bfloat16()
    send = x.repeat_interleave(K, dim=0)[order].contiguous()   # [T*K, H] grouped by destination
    recv_m = torch.empty(sum(out_split), H, device=dev, dtype=torch.bfloat16)
    recv_n = torch.empty_like(recv_m)
    back_m = torch.empty_like(send)
    back_n = torch.empty_like(send)

    def dispatch_m():
        dist.all_to_all_single(recv_m, send, out_split, in_split)

    def dispatch_n():
        dist.all_to_all_single(recv_n, send, out_split, in_split, group=nccl)

    def combine_m():
        dist.all_to_all_single(back_m, recv_m, in_split, out_split)

    def combine_n():
        dist.all_to_all_single(back_n, recv_n, in_split, out_split, group=nccl)

    dispatch_m(); dispatch_n(); combine_m(); combine_n()
    torch.cuda.synchronize()
    ok = bool(torch.equal(recv_m, recv_n)) and bool(torch.equal(back_m, send)) and bool(torch.equal(back_n, send))
    bar_m = lambda: dist.barrier()  # noqa: E731
    bar_n = lambda: dist.barrier(group=nccl)  # noqa: E731
    res = {"world": world, "tokens_per_gpu": T, "hidden": H, "experts": E, "topk": K, "matches_nccl": ok,
           "send_rows_min": min(in_split), "send_rows_max": max(in_split)}
    res["dispatch_moodist_ms"] = timed(dispatch_m, bar_m, args.warmup, args.iters, dev)
    res["dispatch_nccl_ms"] = timed(dispatch_n, bar_n, args.warmup, args.iters, dev)
    res["combine_moodist_ms"] = timed(combine_m, bar_m, args.warmup, args.iters, dev)
    res["combine_nccl_ms"] = timed(combine_n, bar_n, args.warmup, args.iters, dev)
    remote_bytes = (sum(in_split) - in_split[rank]) * H * 2
    res["dispatch_moodist_gbs"] = remote_bytes / res["dispatch_moodist_ms"] / 1e6
    res["dispatch_nccl_gbs"] = remote_bytes / res["dispatch_nccl_ms"] / 1e6
    del send, recv_m, recv_n, back_m, back_n, x, logits
    torch.cuda.empty_cache()

    # ---- reshard: (2 x world/2) blocks -> row shards ----
    R, C = args.reshard_rows, args.reshard_cols
    if world % 2 == 0 and world >= 2:
        pr, pc = 2, world // 2
        br, bc = R // pr, C // pc
        bi, bj = rank // pc, rank % pc
        torch.manual_seed(99)
        rows = R // world
        src_box = {"offset": [bi * br, bj * bc], "shape": [br, bc]}
        dst_box = {"offset": [rank * rows, 0], "shape": [rows, C]}
        op = moodist_b200.compile_op(pg, shape=(R, C), dtype=torch.bfloat16, inputs=[src_box], outputs=[dst_box])
        blk = (torch.arange(br * bc, device=dev, dtype=torch.float32).view(br, bc) % 251 + rank).bfloat16()
        out = torch.empty(rows, C, device=dev, dtype=torch.bfloat16)
        op([blk], [out]).wait()
        # NCCL baseline: gather every block, then slice the rows this rank wants
        allb = torch.empty(world, br, bc, device=dev, dtype=torch.bfloat16)

        def reshard_nccl():
            dist.all_gather_into_tensor(allb, blk, group=nccl)
            full_rows = torch.cat([allb[(rank * rows // br) * pc + j][(rank * rows) % br:(rank * rows) % br + rows] for j in range(pc)], dim=1)
            return full_rows

        ref = reshard_nccl()
        torch.cuda.synchronize()
        res["reshard_matches"] = bool(torch.equal(out, ref))
        res["reshard_moodist_ms"] = timed(lambda: op([blk], [out]), bar_m, args.warmup, args.iters, dev)
        res["reshard_nccl_ms"] = timed(reshard_nccl, bar_n, args.warmup, args.iters, dev)
        res["reshard_pieces"] = op.num_pieces()
    if rank == 0:
        print(json.dumps(res), flush=True)
        if args.out:
            open(args.out, "w").write(json.dumps(res) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
