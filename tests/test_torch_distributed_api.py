"""The torch.distributed surface a user of the backend touches beyond the flat collectives, on CPU ranks:
sub-groups, object collectives, asynchronous works and futures, list forms (even and uneven), rooted
collectives, point-to-point in all its spellings, every dtype and reduce operation, empty tensors, wrong
arguments that must raise before anything is sent, and a second group after the first was destroyed."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _surface(rank, world, port):
    dist = init_moodist(rank, world, port)

    # ---- sub-groups over some of the ranks ----
    g01 = dist.new_group(ranks=[0, 1])
    g12 = dist.new_group(ranks=[1, 2])
    if rank in (0, 1):
        t = torch.full((5,), float(rank + 1))
        dist.all_reduce(t, group=g01)
        assert t.tolist() == [3.0] * 5
    if rank in (1, 2):
        t = torch.full((5,), float(rank + 1))
        dist.all_reduce(t, group=g12)
        assert t.tolist() == [5.0] * 5

    # ---- object collectives (pickled through byte tensors by torch) ----
    out = [None] * world
    dist.all_gather_object(out, {"r": rank, "s": "x" * (rank * 10)})
    assert [o["r"] for o in out] == list(range(world)) and out[2]["s"] == "x" * 20
    objs = [{"a": 1}, 5] if rank == 0 else [None, None]
    dist.broadcast_object_list(objs, src=0)
    assert objs == [{"a": 1}, 5]
    got = [None] * world if rank == 1 else None
    dist.gather_object(rank * 2, got, dst=1)
    if rank == 1:
        assert got == [2 * r for r in range(world)]
    one = [None]
    dist.scatter_object_list(one, [f"s{i}" for i in range(world)] if rank == 0 else None, src=0)
    assert one[0] == f"s{rank}"

    # ---- asynchronous works ----
    t = torch.ones(1000) * (rank + 1)
    w = dist.all_reduce(t, async_op=True)
    w.wait()
    assert float(t[0]) == sum(range(1, world + 1))
    t2 = torch.ones(10)
    w = dist.all_reduce(t2, async_op=True)
    w.get_future().wait()
    assert float(t2[0]) == world and w.is_completed()

    # ---- list forms ----
    outs = [torch.empty(3) for _ in range(world)]
    dist.all_gather(outs, torch.full((3,), float(rank)))
    assert [float(o[0]) for o in outs] == [float(r) for r in range(world)]
    # every rank contributes a different amount
    outs = [torch.full((r + 1, 2), -1.0) for r in range(world)]
    dist.all_gather(outs, torch.full((rank + 1, 2), float(rank)))
    for r, o in enumerate(outs):
        assert o.shape == (r + 1, 2) and bool((o == float(r)).all())
    o2 = torch.empty(2)
    dist.reduce_scatter(o2, [torch.full((2,), float(rank + i)) for i in range(world)])
    assert float(o2[0]) == sum(r + rank for r in range(world))
    ins = [torch.full((2,), float(rank * 10 + d)) for d in range(world)]
    outs = [torch.empty(2) for _ in range(world)]
    dist.all_to_all(outs, ins)
    assert [float(o[0]) for o in outs] == [float(s * 10 + rank) for s in range(world)]

    # ---- coalesced forms, the coalescing manager, functional collectives ----
    pair = [torch.ones(3), torch.ones(5)]
    dist.all_reduce_coalesced(pair)
    assert float(pair[1][0]) == world
    lists = [[torch.empty(3) for _ in range(world)], [torch.empty(2) for _ in range(world)]]
    dist.all_gather_coalesced(lists, [torch.full((3,), float(rank)), torch.full((2,), float(rank))])
    assert float(lists[1][world - 1][0]) == world - 1 and float(lists[0][1][2]) == 1.0
    a, b = torch.ones(4), torch.ones(8) * 2
    with dist._coalescing_manager(device=torch.device("cpu")):
        dist.all_reduce(a)
        dist.all_reduce(b)
    assert float(a[0]) == world and float(b[0]) == 2 * world
    import torch.distributed._functional_collectives as funcol

    assert float(funcol.all_reduce(torch.ones(4), "sum", dist.group.WORLD)[0]) == world
    assert funcol.all_gather_tensor(torch.full((2,), float(rank)), 0, dist.group.WORLD).shape == (2 * world,)
    assert float(funcol.reduce_scatter_tensor(torch.ones(2 * world), "avg", 0, dist.group.WORLD)[0]) == 1.0
    assert float(funcol.all_to_all_single(torch.arange(world, dtype=torch.float32), None, None, dist.group.WORLD)[0]) == rank

    # ---- rooted collectives ----
    t = torch.full((4,), float(rank + 1))
    dist.reduce(t, dst=1)
    if rank == 1:
        assert float(t[0]) == sum(range(1, world + 1))
    g = [torch.empty(2) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.full((2,), float(rank)), g, dst=0)
    if rank == 0:
        assert [float(x[0]) for x in g] == [float(r) for r in range(world)]
    o = torch.empty(2)
    dist.scatter(o, [torch.full((2,), float(i)) for i in range(world)] if rank == 0 else None, src=0)
    assert float(o[0]) == float(rank)

    # ---- point to point ----
    if rank == 0:
        dist.send(torch.arange(10.0), dst=1, tag=3)
        dist.isend(torch.arange(5.0), dst=1).wait()
    elif rank == 1:
        t = torch.empty(10)
        dist.recv(t, src=0, tag=3)
        assert float(t[9]) == 9.0
        t = torch.empty(5)
        dist.irecv(t, src=0).wait()
        assert float(t[4]) == 4.0
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    a, b = torch.full((4,), float(rank)), torch.empty(4)
    for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, a, nxt), dist.P2POp(dist.irecv, b, prv)]):
        w.wait()
    assert float(b[0]) == float(prv)

    # ---- dtypes and reduce operations ----
    for dt in (torch.float64, torch.int32, torch.int64, torch.bfloat16, torch.float16, torch.uint8, torch.int8, torch.int16):
        t = torch.ones(17, dtype=dt)
        dist.all_reduce(t)
        assert float(t.float()[0]) == world and float(t.float()[16]) == world, dt
    flags = torch.ones(17, dtype=torch.bool)
    gathered = torch.empty(17 * world, dtype=torch.bool)
    dist.all_gather_into_tensor(gathered, flags)
    assert bool(gathered.all())
    t = torch.tensor([rank + 1.0, 5.0 - rank])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.tolist() == [float(world), 5.0]
    t = torch.tensor([rank + 1.0])
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    assert t.tolist() == [1.0]
    t = torch.tensor([2.0, float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.PRODUCT)
    assert t.tolist() == [2.0**world, 6.0]
    t = torch.tensor([3.0], dtype=torch.bfloat16)
    dist.all_reduce(t, op=dist.ReduceOp.PRODUCT)
    assert float(t[0]) == 27.0
    bits = torch.tensor([1 << rank, 7, rank], dtype=torch.int64)
    t = bits.clone()
    dist.all_reduce(t, op=dist.ReduceOp.BOR)
    assert t.tolist() == [7, 7, 3]
    t = bits.clone()
    dist.all_reduce(t, op=dist.ReduceOp.BAND)
    assert t.tolist() == [0, 7, 0]
    t = bits.to(torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.BXOR)
    assert t.tolist() == [7, 7, 0 ^ 1 ^ 2]
    out = torch.empty(2, dtype=torch.uint8)
    dist.reduce_scatter_tensor(out, torch.full((2 * world,), 1 << rank, dtype=torch.uint8), op=dist.ReduceOp.BOR)
    assert out.tolist() == [7, 7]
    # bool tensors keep bytes 0 / 1: their sum is "any", their product "all"; complex numbers reduce as pairs of reals
    anyone = torch.tensor([True, False, rank == 0, rank == 1])
    dist.all_reduce(anyone)
    assert anyone.tolist() == [True, False, True, True] and anyone.view(torch.uint8).tolist() == [1, 0, 1, 1]
    everyone = torch.tensor([True, False, rank == 0, rank != 5])
    dist.all_reduce(everyone, op=dist.ReduceOp.PRODUCT)
    assert everyone.tolist() == [True, False, False, True]
    z = torch.full((4,), complex(rank + 1, -rank))
    dist.all_reduce(z)
    assert z[0] == complex(sum(range(1, world + 1)), -sum(range(world)))

    # ---- empty tensors ----
    dist.all_reduce(torch.empty(0))
    dist.all_gather_into_tensor(torch.empty(0), torch.empty(0))
    dist.broadcast(torch.empty(0), src=0)

    # ---- wrong arguments raise on the rank that passed them, and the group stays usable ----
    with pytest.raises(RuntimeError, match="contiguous"):
        dist.all_reduce(torch.ones(8, 8)[:, ::2])
    with pytest.raises(RuntimeError, match="unsupported reduce op"):
        dist.all_reduce(torch.ones(3), op=dist.ReduceOp.BAND)  # bitwise on a float
    with pytest.raises(RuntimeError, match="elements but this rank's input"):
        dist.all_gather([torch.empty(4) for _ in range(world)], torch.ones(3))
    with pytest.raises(RuntimeError, match="world_size x output"):
        dist.reduce_scatter_tensor(torch.empty(2), torch.ones(2 * world + 1))
    if rank == 0:
        with pytest.raises(RuntimeError, match="scatter inputs"):
            dist.scatter(torch.empty(2), [torch.ones(3) for _ in range(world)], src=0)
    t = torch.ones(4)
    dist.all_reduce(t)
    assert t.tolist() == [float(world)] * 4

    dist.barrier()
    dist.destroy_process_group()

    # ---- a new default group in the same processes ----
    dist = init_moodist(rank, world, port + 7)
    t = torch.ones(3)
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.barrier()
    dist.destroy_process_group()


def test_torch_distributed_surface_world3():
    run_ranks(_surface, 3, timeout=240)


def _wrappers(rank, world, port):
    """torch's own parallel wrappers running over the backend: DDP, ZeroRedundancyOptimizer, DTensor, fully_shard,
    distributed checkpointing, tensor parallelism, pipeline schedules."""
    dist = init_moodist(rank, world, port)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.optim import ZeroRedundancyOptimizer
    from torch.distributed.tensor import Replicate, Shard, distribute_tensor
    from torch.nn.parallel import DistributedDataParallel as DDP

    def same_everywhere(module):
        flat = torch.cat([p.detach().reshape(-1) for p in module.parameters()])
        outs = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(outs, flat)
        return all(torch.equal(o, outs[0]) for o in outs)

    # DDP: different data per rank, identical parameters after every step, equal to the single-process update
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    oracle = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    oracle.load_state_dict(net.state_dict())
    ddp = DDP(net)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
    oopt = torch.optim.SGD(oracle.parameters(), lr=0.1)
    for step in range(3):
        xs = [torch.randn(8, 16, generator=torch.Generator().manual_seed(r * 10 + step)) for r in range(world)]
        ddp(xs[rank]).sum().backward()
        opt.step()
        opt.zero_grad()
        (sum(oracle(x).sum() for x in xs) / world).backward()
        oopt.step()
        oopt.zero_grad()
    assert same_everywhere(net)
    for p, q in zip(net.parameters(), oracle.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)

    # ZeRO-1 optimizer wrapper
    lin = torch.nn.Linear(8, 8)
    for p in lin.parameters():
        dist.broadcast(p.data, 0)
    zopt = ZeroRedundancyOptimizer(lin.parameters(), optimizer_class=torch.optim.SGD, lr=0.1)
    lin(torch.ones(2, 8)).sum().backward()
    for p in lin.parameters():
        dist.all_reduce(p.grad)
    zopt.step()
    assert same_everywhere(lin)

    # DTensor: shard, replicate, re-shard along the other dimension, reduce
    mesh = init_device_mesh("cpu", (world,))
    full = torch.arange(world * 4 * 6, dtype=torch.float32).view(world * 4, 6)
    dt = distribute_tensor(full, mesh, [Shard(0)])
    assert torch.equal(dt.to_local(), full[rank * 4 : (rank + 1) * 4])
    assert torch.equal(dt.redistribute(mesh, [Replicate()]).to_local(), full)
    assert torch.equal(dt.redistribute(mesh, [Shard(1)]).full_tensor(), full)
    assert float((dt * 2).sum().full_tensor()) == float(full.sum() * 2)

    # fully_shard (FSDP2) on CPU parameters: all_gather_into_tensor / reduce_scatter_tensor under torch's schedule
    torch.manual_seed(1)
    fs = torch.nn.Sequential(torch.nn.Linear(12, 24), torch.nn.Linear(24, 6))
    ref = torch.nn.Sequential(torch.nn.Linear(12, 24), torch.nn.Linear(24, 6))
    ref.load_state_dict(fs.state_dict())
    fully_shard(fs, mesh=mesh)
    fopt = torch.optim.SGD(fs.parameters(), lr=0.1)
    xs = [torch.randn(4, 12, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
    fs(xs[rank]).sum().backward()
    fopt.step()
    (sum(ref(x).sum() for x in xs) / world).backward()
    with torch.no_grad():
        for p in ref.parameters():
            p -= 0.1 * p.grad
    for p, q in zip(fs.parameters(), ref.parameters()):
        torch.testing.assert_close(p.full_tensor(), q, rtol=1e-5, atol=1e-6)

    # torch.distributed.checkpoint: saved sharded by rows, loaded sharded by columns
    import shutil
    import tempfile

    import torch.distributed.checkpoint as dcp

    where = [tempfile.mkdtemp(prefix="moodist-dcp-") if rank == 0 else None]
    dist.broadcast_object_list(where, src=0)
    table = torch.arange(24.0).view(6, 4)
    dcp.save({"w": distribute_tensor(table, mesh, [Shard(0)]), "step": torch.tensor(7)}, checkpoint_id=where[0])
    loaded = {"w": distribute_tensor(torch.zeros(6, 4), mesh, [Shard(1)]), "step": torch.tensor(0)}
    dcp.load(loaded, checkpoint_id=where[0])
    assert torch.equal(loaded["w"].full_tensor(), table) and int(loaded["step"]) == 7
    dist.barrier()
    if rank == 0:
        shutil.rmtree(where[0], ignore_errors=True)

    # tensor parallelism through DTensor: column-parallel up, row-parallel down, forward and backward
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up = torch.nn.Linear(16, 32)
            self.down = torch.nn.Linear(32, 16)

        def forward(self, x):
            return self.down(torch.relu(self.up(x)))

    torch.manual_seed(5)
    whole_mlp, split_mlp = MLP(), MLP()
    split_mlp.load_state_dict(whole_mlp.state_dict())
    split_mlp = parallelize_module(split_mlp, mesh, {"up": ColwiseParallel(), "down": RowwiseParallel()})
    x = torch.randn(4, 16, generator=torch.Generator().manual_seed(6))
    y_split, y_whole = split_mlp(x), whole_mlp(x)
    y_split.sum().backward()
    y_whole.sum().backward()
    torch.testing.assert_close(y_split, y_whole, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(split_mlp.up.weight.grad.full_tensor(), whole_mlp.up.weight.grad, rtol=1e-5, atol=1e-5)

    # torch.distributed.pipelining: one layer per rank, GPipe and 1F1B schedules (receives are posted before sends)
    from torch.distributed.pipelining import PipelineStage, Schedule1F1B, ScheduleGPipe

    torch.manual_seed(3)
    layers = [torch.nn.Linear(8, 8) for _ in range(world)]
    stage = PipelineStage(layers[rank], rank, world, torch.device("cpu"))
    batch = torch.randn(8, 8, generator=torch.Generator().manual_seed(4))
    for schedule_class in (ScheduleGPipe, Schedule1F1B):
        schedule = schedule_class(stage, n_microbatches=4, loss_fn=lambda y, t: ((y - t) ** 2).mean())
        losses = []
        if rank == 0:
            schedule.step(batch)
        elif rank == world - 1:
            schedule.step(target=torch.zeros(8, 8), losses=losses)
        else:
            schedule.step()
        if rank == world - 1:
            whole = batch
            for layer in layers:
                whole = layer(whole)
            want = [(chunk**2).mean().item() for chunk in whole.chunk(4)]
            assert all(abs(a.item() - b) < 1e-5 for a, b in zip(losses, want)), (losses, want)
        dist.barrier()

    dist.barrier()
    dist.destroy_process_group()


def test_torch_parallel_wrappers_over_the_backend_world2():
    run_ranks(_wrappers, 2, timeout=240)


def _threads(rank, world, port):
    """Three groups over the same ranks, each driven by its own thread from its very first operation on."""
    import threading

    dist = init_moodist(rank, world, port)
    g1 = dist.new_group(ranks=list(range(world)))
    g2 = dist.new_group(ranks=list(range(world)))
    errors = []

    def loop(group, base):
        try:
            for i in range(200):
                t = torch.full((257,), float(base + i + rank))
                dist.all_reduce(t, group=group)
                want = sum(base + i + r for r in range(world))
                assert float(t[0]) == want and float(t[-1]) == want
                out = torch.empty(world * 33)
                dist.all_gather_into_tensor(out, torch.full((33,), float(rank + i)), group=group)
                assert float(out[33 * (world - 1)]) == world - 1 + i
        except Exception as e:  # reported by the main thread
            errors.append(repr(e))

    workers = [threading.Thread(target=loop, args=(g1, 0)), threading.Thread(target=loop, args=(g2, 1000))]
    for t in workers:
        t.start()
    loop(None, 5000)  # the default group, from the main thread, at the same time
    for t in workers:
        t.join()
    assert not errors, errors[:2]
    dist.barrier()
    dist.destroy_process_group()


def test_groups_driven_from_separate_threads_world3():
    run_ranks(_threads, 3, timeout=240)
