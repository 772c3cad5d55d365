"""CPU-rank benchmark of the host engine: collectives on CPU tensors, the queue, the store and compile_op.

    python benchmarks/host_collectives.py --world 2 --mib 4 64 --gloo

Spawns ``--world`` processes on this machine (no GPU involved) and prints one line per operation and size:
median and best time over ``--iters`` runs after ``--warmup`` runs (wall clock from a barrier to the return of the
call, maximum over the ranks per run), and the same for gloo when asked.  Environment variables select the transport under test: ``MOODIST_DIRECT_CPU=0`` keeps
payloads on the sockets, ``MOODIST_DISABLE_UNIX_SOCKETS=1`` uses loopback TCP, ``MOODIST_SPIN_US=0`` lets threads
sleep at once.  The reference has no CPU-only mode to compare with (its groups need a GPU and refuse loopback:
``core/group.cc:68-70``, ``core/setup_comms.cc:129-131``).
"""

from __future__ import annotations

import argparse
import os
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from moodist_b200.utils.testing import init_moodist, run_ranks  # noqa: E402


def _time(dist, fn, warmup, iters):
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(iters):
        dist.barrier()
        t0 = time.perf_counter()
        fn()
        samples.append(time.perf_counter() - t0)
    dist.barrier()
    # an operation is over when its slowest rank is done: per-iteration maximum over the ranks
    t = torch.tensor(samples, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    samples = t.tolist()
    return statistics.median(samples), min(samples)


def _rank(rank, world, port, backend, sizes_mib, warmup, iters, extras):
    import torch.distributed as dist

    if backend == "moodist":
        dist = init_moodist(rank, world, port)
    else:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rows = []
    # the average is what sharded training asks for; gloo has none, so it is timed on the sum
    rs_op, rs_name = (dist.ReduceOp.AVG, "avg") if backend == "moodist" else (dist.ReduceOp.SUM, "sum")
    for mib in sizes_mib:
        n = int(mib * (1 << 20)) // 4
        n -= n % world
        x = torch.randn(n)
        out = torch.empty(world * n)
        o = torch.empty(n // world)
        its = max(3, iters // 4) if mib >= 64 else iters
        for name, fn, moved in (
            ("all_reduce", lambda: dist.all_reduce(x), 2 * n * 4 * (world - 1) / world),
            ("all_gather", lambda: dist.all_gather_into_tensor(out, x), n * 4 * (world - 1)),
            ("reduce_scatter " + rs_name, lambda: dist.reduce_scatter_tensor(o, x, op=rs_op), n * 4 * (world - 1) / world),
            ("broadcast", lambda: dist.broadcast(x, 0), n * 4),
        ):
            med, best = _time(dist, fn, warmup, its)
            rows.append((f"{name} {mib:g} MiB fp32", med, best, moved))
    if world >= 2:
        # point to point between ranks 0 and 1: from the barrier until the receiver has the tensor
        for mib in [1 / 1024] + list(sizes_mib):
            n = max(1, int(mib * (1 << 20)) // 4)
            x, y = torch.randn(n), torch.empty(n)

            def exchange():
                if rank == 0:
                    dist.send(x, 1)
                elif rank == 1:
                    dist.recv(y, 0)

            med, best = _time(dist, exchange, warmup, max(3, iters // 4) if mib >= 64 else iters)
            size = f"{mib:g} MiB" if mib >= 1 else f"{mib * 1024:g} KiB"
            rows.append((f"send -> recv {size} fp32", med, best, n * 4))
    small = torch.ones(16)
    med, best = _time(dist, lambda: dist.all_reduce(small), warmup * 5, iters * 10)
    rows.append(("all_reduce 16 elements", med, best, 0))
    med, best = _time(dist, dist.barrier, 0, iters * 10)
    rows.append(("barrier", med, best, 0))

    if backend == "moodist" and extras:
        import moodist_b200 as moodist

        pg = moodist.get_backend(device="cpu")
        q = moodist.Queue(pg, location=0, name="bench")
        count = 1000
        items = [torch.full((256,), i, dtype=torch.int64) for i in range(count)]
        dist.barrier()
        if rank == world - 1:
            t0 = time.perf_counter()
            for t in items:
                q.put_tensor(t)
            rows.append(("queue put int64[256] (to rank 0)", (time.perf_counter() - t0) / count, 0.0, 0))
        if rank == 0:
            t0 = time.perf_counter()
            for _ in range(count):
                q.get_tensor(timeout=60)
            rows.append(("queue get int64[256] (fed by the last rank)", (time.perf_counter() - t0) / count, 0.0, 0))
        dist.barrier()
        if rank == 0:
            for t in items:
                q.put_tensor(t)
            time.sleep(0.1)
            t0 = time.perf_counter()
            for _ in range(count):
                q.get_tensor()
            rows.append(("queue get, items already there", (time.perf_counter() - t0) / count, 0.0, 0))
        dist.barrier()
        m = 4096 - 4096 % world
        r = m // world
        full_rows = torch.randn(r, m)
        dst = torch.empty(m, r)
        op = moodist.compile_op(pg, shape=(m, m), dtype=torch.float32, inputs=[{"offset": [rank * r, 0], "shape": [r, m]}],
                                outputs=[{"offset": [0, rank * r], "shape": [m, r]}])
        med, best = _time(dist, lambda: op([full_rows], [dst]).wait(), 2, max(3, iters // 2))
        rows.append((f"compile_op rows -> columns [{m}, {m}] fp32", med, best, 0))
        stats = pg.host_stats()
        if rank == 0:
            print(f"# transport: {stats}", flush=True)
    if rank in (0, world - 1):
        for label, med, best, moved in rows:
            if rank != 0 and "queue put" not in label:
                continue
            bw = f"  {moved / med / 2**30:6.2f} GiB/s per rank" if moved else ""
            unit = 1e3 if med >= 1e-3 else 1e6
            print(f"{backend:8s} world {world}  {label:46s} {med * unit:9.2f} {'ms' if unit == 1e3 else 'us'}"
                  f" (best {best * unit:8.2f}){bw}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--mib", type=float, nargs="+", default=[4.0], help="tensor sizes in MiB (fp32)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--gloo", action="store_true", help="also time torch's gloo backend in the same harness")
    ap.add_argument("--no-extras", action="store_true", help="collectives only (no queue, compile_op)")
    args = ap.parse_args()
    run_ranks(_rank, args.world, "moodist", args.mib, args.warmup, args.iters, not args.no_extras, timeout=900)
    if args.gloo:
        run_ranks(_rank, args.world, "gloo", args.mib, args.warmup, args.iters, False, timeout=900)


if __name__ == "__main__":
    main()
