"""What tests/test_sanitizers.py runs against the instrumented copy of the package (every native line of the
serializer, the torch bindings and the core compiled with a sanitizer): the serializer on random objects and on
damaged streams, then three CPU ranks going through collectives, point-to-point, the queue and compile_op.
Prints SCENARIO OK at the end; a finding of the sanitizer ends the process with its own exit code first."""

import collections
import dataclasses
import datetime
import random
import re
import sys

import torch

import moodist_b200 as moodist
from moodist_b200.utils.testing import init_moodist, run_ranks


@dataclasses.dataclass
class Record:
    a: int
    b: list


class Slots:
    __slots__ = ("a",)

    def __init__(self):
        self.a = [1]


def _random_object(rng, depth=0):
    r = rng.random()
    if depth > 4 or r < 0.3:
        return rng.choice([None, True, 1, -5, 2**70, 1.5, "s", "é" * 3, b"b", bytearray(b"x"), (), [], {}, frozenset(),
                           Record(1, [2]), Slots(), re.compile("a"), datetime.date(2020, 1, 1), Ellipsis, int, len,
                           collections.OrderedDict(a=1), collections.deque([1], maxlen=3)])
    if r < 0.5:
        return [_random_object(rng, depth + 1) for _ in range(rng.randint(0, 5))]
    if r < 0.65:
        return tuple(_random_object(rng, depth + 1) for _ in range(rng.randint(0, 5)))
    if r < 0.8:
        return {rng.choice(["a", "b", 1, (1, 2), "longer key"]): _random_object(rng, depth + 1) for _ in range(rng.randint(0, 5))}
    if r < 0.9:
        x = [_random_object(rng, depth + 1)]
        x.append(x)
        return x
    shared = _random_object(rng, depth + 1)
    return [shared, shared, {"again": shared}]


def serializer(rounds):
    rng = random.Random(7)
    for _ in range(rounds):
        blob = bytes(moodist.serialize(_random_object(rng)).numpy())
        moodist.deserialize(torch.frombuffer(bytearray(blob), dtype=torch.uint8))
        for _ in range(3):  # damaged and cut streams may raise, nothing more
            damaged = bytearray(blob)
            damaged[rng.randrange(len(damaged))] = rng.randrange(256)
            for candidate in (damaged, damaged[: rng.randrange(len(damaged) + 1)]):
                try:
                    moodist.deserialize(bytes(candidate))
                except Exception:  # noqa: BLE001
                    pass
    for refused in (lambda: 1, (i for i in ())):
        try:
            moodist.serialize(refused)
        except (TypeError, ValueError):
            pass


def _ranks(rank, world, port):
    dist = init_moodist(rank, world, port)
    pg = moodist.get_backend(device="cpu")
    for n in (1, 1000, (1 << 18) + 1):
        x = torch.full((n,), float(rank))
        dist.all_reduce(x)
        assert float(x[-1]) == world * (world - 1) / 2
        out = torch.empty(world * n)
        dist.all_gather_into_tensor(out, torch.full((n,), float(rank)))
        assert float(out[-1]) == world - 1
        o = torch.empty(n, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o, torch.ones(world * n, dtype=torch.bfloat16), op=dist.ReduceOp.AVG)
        assert float(o[0]) == 1.0
        dist.broadcast(x, src=world - 1)
    outs = [torch.empty(r + 1) for r in range(world)]
    dist.all_gather(outs, torch.full((rank + 1,), float(rank)))
    assert [float(o[0]) for o in outs] == [float(r) for r in range(world)]
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = torch.empty(300)
    for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, got, prv), dist.P2POp(dist.isend, torch.full((300,), float(rank)), nxt)]):
        w.wait()
    assert float(got[0]) == prv
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "payload": "x" * rank})
    assert [g["rank"] for g in gathered] == list(range(world))
    q = moodist.Queue(pg, location=0, name="scenario")
    q.put_object(("hello", rank))
    q.put_tensor(torch.full((70000,), float(rank))).wait()  # too large to travel inside its message
    if rank == 0:
        items = [q.get_tensor(timeout=60) for _ in range(2 * world)]  # objects arrive as their uint8 encoding
        assert sorted(t.numel() for t in items if t.dtype == torch.float32) == [70000] * world
        assert sorted(moodist.deserialize(t)[1] for t in items if t.dtype == torch.uint8) == list(range(world))
    dist.barrier()
    with q.transaction() as tx:
        tx.put_object("in a transaction")
        tx.put_object(rank)
    if rank == 0:
        assert sorted(str(q.get_object(timeout=60)) for _ in range(2 * world)).count("in a transaction") == world
    everywhere = moodist.Queue(pg, location=range(world), name="scenario-multicast")
    if rank == 1:
        everywhere.put_object("to all")
    assert everywhere.get_object(timeout=60) == "to all"
    rows = 8
    op = moodist.compile_op(pg, shape=(rows * world, rows * world), dtype=torch.float32,
                            inputs=[{"offset": [rank * rows, 0], "shape": [rows, rows * world]}],
                            outputs=[{"offset": [0, rank * rows], "shape": [rows * world, rows]}])
    full = torch.arange((rows * world) ** 2, dtype=torch.float32).view(rows * world, rows * world)
    dst = torch.empty(rows * world, rows)
    op([full[rank * rows : (rank + 1) * rows].contiguous()], [dst]).wait()
    assert torch.equal(dst, full[:, rank * rows : (rank + 1) * rows])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    serializer(int(sys.argv[1]) if len(sys.argv) > 1 else 300)
    run_ranks(_ranks, 3, timeout=600)
    print("SCENARIO OK", moodist.__file__)
