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
