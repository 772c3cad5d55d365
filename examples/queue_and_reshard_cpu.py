"""Two CPU ranks over the moodist backend: a work queue fed by rank 1 and drained by rank 0, then a compiled
row-sharded -> column-sharded redistribution of a matrix. Runs anywhere (no GPU needed):

    python examples/queue_and_reshard_cpu.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moodist_b200.utils.testing import init_moodist, run_ranks  # noqa: E402


def main(rank, world, port):
    dist = init_moodist(rank, world, port)  # torch.distributed with backend "moodist"
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")

    # ---- a queue that lives on rank 0; anybody may put, rank 0 gets ----
    q = moodist.Queue(pg, location=0, name="work")
    if rank == 1:
        for i in range(5):
            q.put_object({"job": i, "payload": torch.full((4,), float(i))})
        with q.transaction() as tx:  # both items become visible together
            tx.put_object("last-a")
            tx.put_object("last-b")
    else:
        jobs = [q.get_object() for _ in range(5)]
        assert [j["job"] for j in jobs] == list(range(5))
        assert (q.get_object(), q.get_object()) == ("last-a", "last-b")
        print(f"rank 0 drained the queue: {len(jobs)} jobs + a transaction of 2")
    dist.barrier()

    # ---- compile a redistribution once, run it many times ----
    n = 1024
    rows = n // world
    op = moodist.compile_op(pg, shape=(n, n), dtype=torch.float32,
                            inputs=[{"offset": (rank * rows, 0), "shape": (rows, n)}],    # I hold these rows
                            outputs=[{"offset": (0, rank * rows), "shape": (n, rows)}])   # I want these columns
    full = torch.arange(n * n, dtype=torch.float32).view(n, n)
    mine = full[rank * rows:(rank + 1) * rows].contiguous()
    cols = torch.empty(n, rows)
    op([mine], [cols]).wait()
    assert torch.equal(cols, full[:, rank * rows:(rank + 1) * rows])
    if rank == 0:
        print(f"resharded a [{n}, {n}] matrix from rows to columns with {op.num_pieces()} strided pieces per rank")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    run_ranks(main, 2, timeout=120)
    print("ok")
