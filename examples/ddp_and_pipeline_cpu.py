"""torch's own wrappers over the moodist backend on CPU ranks: DistributedDataParallel training a small model, then
a three-stage pipeline that hands activations from rank to rank with receives posted before the sends.  Runs
anywhere (no GPU needed):

    python examples/ddp_and_pipeline_cpu.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moodist_b200.utils.testing import init_moodist, run_ranks  # noqa: E402


def main(rank, world, port):
    dist = init_moodist(rank, world, port)  # torch.distributed with backend "moodist"
    from torch.nn.parallel import DistributedDataParallel as DDP

    # ---- data parallel: every rank sees its own batches, gradients are averaged through the backend ----
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 64), torch.nn.Tanh(), torch.nn.Linear(64, 1))
    ddp = DDP(model)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    target = torch.nn.Linear(16, 1)
    torch.nn.init.constant_(target.weight, 0.3)
    losses = []
    for step in range(30):
        x = torch.randn(32, 16, generator=torch.Generator().manual_seed(1000 * rank + step))
        loss = torch.nn.functional.mse_loss(ddp(x), target(x).detach())
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    copies = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(copies, flat)
    assert all(torch.equal(c, copies[0]) for c in copies), "replicas diverged"
    if rank == 0:
        print(f"DDP over {world} ranks: loss {losses[0]:.3f} -> {losses[-1]:.3f}, replicas identical")

    # ---- pipeline: stage r multiplies by (r + 2); micro-batches flow 0 -> 1 -> ... -> last ----
    micro_batches = 4
    results = []
    for m in range(micro_batches):
        work = None
        inbox = torch.empty(8)
        if rank > 0:
            work = dist.irecv(inbox, src=rank - 1, tag=m)  # posted first: returns at once
        x = torch.full((8,), float(m + 1)) if rank == 0 else None
        if work is not None:
            work.wait()
            x = inbox
        y = x * (rank + 2)
        if rank < world - 1:
            dist.isend(y, dst=rank + 1, tag=m).wait()
        else:
            results.append(float(y[0]))
    if rank == world - 1:
        factor = 1
        for r in range(world):
            factor *= r + 2
        assert results == [float((m + 1) * factor) for m in range(micro_batches)], results
        print(f"pipeline of {world} stages: {results}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    run_ranks(main, 3, timeout=120)
    print("ok")
