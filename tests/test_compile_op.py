"""compile_op on CPU ranks: the patterns of the reference's tests/test_compile_op.py (p2p, broadcast,
gather, scatter, all-gather, 2-D shapes, multiple inputs, dtypes, reuse, ranks without inputs/outputs) plus
strided reshards (row-sharded -> column-sharded [4096, 4096] fp32) checked against a single-process oracle."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _global(shape, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = 1
    for s in shape:
        n *= s
    if dtype in (torch.int32, torch.int64):
        return torch.randint(-1000, 1000, shape, generator=g, dtype=dtype)
    return torch.randn(n, generator=g).view(shape).to(dtype)


def _cut(full, box):
    sl = tuple(slice(o, o + s) for o, s in zip(box["offset"], box["shape"]))
    return full[sl].contiguous()


def _run(moodist, pg, full, inputs, outputs, device="cpu", repeat=1):
    op = moodist.compile_op(pg, shape=tuple(full.shape), dtype=full.dtype, inputs=inputs, outputs=outputs)
    for it in range(repeat):
        src = full + it
        ins = [_cut(src, b).to(device) for b in (inputs or [])]
        outs = [torch.full(b["shape"], -7, dtype=full.dtype, device=device) for b in (outputs or [])]
        op(ins, outs).wait()
        if device != "cpu":
            torch.cuda.synchronize()
        for o, b in zip(outs, outputs or []):
            assert torch.equal(o.cpu(), _cut(src, b)), (b, it)
    return op


def _patterns(rank, world, port, device):
    dist = init_moodist(rank, world, port, device=device)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device=device)
    dev = "cpu" if device == "cpu" else f"cuda:{rank}"
    last = world - 1
    # point to point: rank 0 -> last rank
    full = _global((64, 16), torch.float32, 1)
    box = {"offset": [0, 0], "shape": [64, 16]}
    _run(moodist, pg, full, [box] if rank == 0 else None, [box] if rank == last else None, dev)
    # broadcast from rank 0
    _run(moodist, pg, full, [box] if rank == 0 else None, [box], dev)
    # gather to rank 0 / scatter from rank 0 / all-gather (row shards)
    rows = 64 // world
    mine = {"offset": [rank * rows, 0], "shape": [rows, 16]}
    whole = {"offset": [0, 0], "shape": [rows * world, 16]}
    _run(moodist, pg, full, [mine], [whole] if rank == 0 else None, dev)
    _run(moodist, pg, full, [whole] if rank == 0 else None, [mine], dev)
    _run(moodist, pg, full, [mine], [whole], dev, repeat=3)  # reuse of the compiled op
    # dtypes
    for dtype in (torch.float64, torch.float16, torch.bfloat16, torch.int32, torch.int64):
        f = _global((8 * world, 6), dtype, 2)
        m = {"offset": [rank * 8, 0], "shape": [8, 6]}
        _run(moodist, pg, f, [m], [{"offset": [0, 0], "shape": [8 * world, 6]}], dev)
    # multiple inputs per rank, 3-D shape, outputs that straddle inputs
    f3 = _global((4 * world, 6, 10), torch.float32, 3)
    ins = [{"offset": [rank * 4, 0, 0], "shape": [2, 6, 10]}, {"offset": [rank * 4 + 2, 0, 0], "shape": [2, 6, 10]}]
    outs = [{"offset": [1, 2, 3], "shape": [4 * world - 2, 3, 5]}]
    _run(moodist, pg, f3, ins, outs, dev)
    # row-sharded -> column-sharded
    n = ((4096 if device == "cpu" else 2048) // world) * world
    fr = _global((n, n), torch.float32, 4)
    r, c = n // world, n // world
    _run(moodist, pg, fr, [{"offset": [rank * r, 0], "shape": [r, n]}], [{"offset": [0, rank * c], "shape": [n, c]}], dev)
    # uneven boxes: per-rank maxima on different sides of the kernel's grid thresholds (1 MiB on rank 0, 512 KiB
    # on the others) and a rank that holds nothing while the others move more than one CTA's worth
    big = _global((384 * world + 128, 512), torch.float32, 5)  # 2 KiB rows
    r0 = 512 if rank == 0 else 256
    lo = 0 if rank == 0 else 512 + (rank - 1) * 256
    total = 512 + (world - 1) * 256
    big = big[:total].contiguous() if big.shape[0] >= total else _global((total, 512), torch.float32, 5)
    cols = 512 // world
    _run(moodist, pg, big, [{"offset": [lo, 0], "shape": [r0, 512]}], [{"offset": [0, rank * cols], "shape": [total, cols]}], dev,
         repeat=2)
    wide = _global((96, 1024), torch.float32, 6)  # 384 KiB in one box
    wbox = {"offset": [0, 0], "shape": [96, 1024]}
    _run(moodist, pg, wide, [wbox] if rank == 0 else None, [wbox] if rank == 1 else None, dev, repeat=2)
    # uncovered output is an error on every rank
    with pytest.raises(RuntimeError, match="no input covers"):
        moodist.compile_op(pg, shape=(4, 4), dtype=torch.float32, inputs=[{"offset": [0, 0], "shape": [2, 4]}] if rank == 0 else None,
                           outputs=[{"offset": [0, 0], "shape": [4, 4]}])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_compile_op_cpu(world):
    run_ranks(_patterns, world, "cpu", timeout=240)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_compile_op_cuda_2gpu():
    run_ranks(_patterns, 2, "cuda", timeout=240, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})


def _planner_body(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    op = moodist.compile_op(pg, shape=(8, 8), dtype=torch.float32,
                            inputs=[{"offset": [rank * 4, 0], "shape": [4, 8]}],
                            outputs=[{"offset": [0, rank * 4], "shape": [8, 4]}])
    pieces = sorted(op.pieces())
    assert len(pieces) == 2
    for src_rank, src_input, dst_output, rows, row_bytes, src_off, src_pitch, dst_off, dst_pitch in pieces:
        assert rows == 4 and row_bytes == 16 and src_pitch == 32 and dst_pitch == 16
        assert src_off == rank * 16 and dst_off == src_rank * 4 * 16
    dist.destroy_process_group()


def test_planner_pieces_are_2d():
    """Row -> column reshard of a [8, 8] tensor over 2 ranks: one strided piece per source."""
    run_ranks(_planner_body, 2, timeout=60)


def _dtensors_and_errors(rank, world, port):
    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Replicate, Shard, distribute_tensor

    pg = moodist.get_backend(device="cpu")
    mesh = init_device_mesh("cpu", (world,))
    full = torch.arange(10 * 6, dtype=torch.float32).view(10, 6)  # 10 rows over 4 ranks: 3, 3, 3, 1

    # DTensors say where this rank's box lies; shape and dtype come from them
    src = distribute_tensor(full, mesh, [Shard(0)])
    dst = distribute_tensor(torch.zeros_like(full), mesh, [Shard(1)])
    op = moodist.compile_op(pg, inputs=[src], outputs=[dst])
    out = torch.empty_like(dst.to_local())
    op([src.to_local().contiguous()], [out]).wait()
    assert torch.equal(out, distribute_tensor(full, mesh, [Shard(1)]).to_local())

    whole = distribute_tensor(torch.zeros_like(full), mesh, [Replicate()])
    op = moodist.compile_op(pg, inputs=[src], outputs=[whole])
    out = torch.empty(10, 6)
    op([src.to_local().contiguous()], [out]).wait()
    assert torch.equal(out, full)

    # blocks of a 2-D mesh -> rows of a 1-D mesh
    mesh2 = init_device_mesh("cpu", (2, world // 2))
    big = torch.arange(8 * 12, dtype=torch.float32).view(8, 12)
    blocks = distribute_tensor(big, mesh2, [Shard(0), Shard(1)])
    rows = distribute_tensor(torch.zeros_like(big), mesh, [Shard(0)])
    op = moodist.compile_op(pg, inputs=[blocks], outputs=[rows])
    out = torch.empty_like(rows.to_local())
    op([blocks.to_local().contiguous()], [out]).wait()
    assert torch.equal(out, distribute_tensor(big, mesh, [Shard(0)]).to_local())

    # malformed descriptions raise on the calling rank, before the collective part
    f32 = torch.float32
    bad_calls = [
        (dict(shape=(4, 4), dtype=f32, inputs=[{"offset": [0, 0]}]), ValueError),
        (dict(shape=(4, 4), dtype=f32, inputs=[{"offset": [0], "shape": [4, 4]}]), ValueError),
        (dict(shape=(4, 4), dtype=f32, inputs=[{"offset": [0, 0.5], "shape": [4, 4]}]), TypeError),
        (dict(shape=(4, 4), dtype="float32", inputs=None), TypeError),
        (dict(dtype=f32, inputs=None), ValueError),
        (dict(shape=(4, 4), dtype=f32, inputs={"offset": [0, 0], "shape": [4, 4]}), TypeError),
    ]
    for kwargs, exc in bad_calls:
        with pytest.raises(exc, match="compile_op"):
            moodist.compile_op(pg, **kwargs)
    with pytest.raises(RuntimeError, match="exceeds the global shape"):
        moodist.compile_op(pg, shape=(4, 4), dtype=f32, inputs=[{"offset": [2, 0], "shape": [4, 4]}], outputs=None)

    # tensors that do not fit the compiled op are refused at call time and the op stays usable
    op = moodist.compile_op(pg, shape=(world * 2, 4), dtype=f32, inputs=[{"offset": [rank * 2, 0], "shape": [2, 4]}],
                            outputs=[{"offset": [0, 0], "shape": [world * 2, 4]}])
    with pytest.raises(RuntimeError, match="elements"):
        op([torch.zeros(3, 4)], [torch.empty(world * 2, 4)]).wait()
    with pytest.raises(RuntimeError, match="dtype"):
        op([torch.zeros(2, 4, dtype=torch.float64)], [torch.empty(world * 2, 4)]).wait()
    out = torch.empty(world * 2, 4)
    op([torch.full((2, 4), float(rank))], [out]).wait()
    assert out[::2, 0].tolist() == [float(r) for r in range(world)]
    dist.barrier()
    dist.destroy_process_group()


def test_compile_op_dtensors_and_argument_errors_world4():
    run_ranks(_dtensors_and_errors, 4, timeout=240)


def _successive_groups(rank, world, port):
    """Four default groups one after the other in the same processes, each used for compile_op and a queue (state a
    subsystem keeps per group must go with the group: the next one may live at the same address)."""
    import moodist_b200 as moodist

    for generation in range(4):
        dist = init_moodist(rank, world, port + generation)
        pg = moodist.get_backend(device="cpu")
        op = moodist.compile_op(pg, shape=(world * 2, 4), dtype=torch.float32,
                                inputs=[{"offset": [rank * 2, 0], "shape": [2, 4]}],
                                outputs=[{"offset": [0, 0], "shape": [world * 2, 4]}])
        out = torch.empty(world * 2, 4)
        op([torch.full((2, 4), float(rank + generation))], [out]).wait()
        assert out[::2, 0].tolist() == [float(r + generation) for r in range(world)]
        q = moodist.Queue(pg, location=0, name="per-generation")
        q.put_object(generation)
        if rank == 0:
            assert sorted(q.get_object(timeout=30) for _ in range(world)) == [generation] * world
        dist.barrier()
        del op, q, pg
        dist.destroy_process_group()


def test_compile_op_and_queue_on_successive_groups():
    run_ranks(_successive_groups, 2, timeout=120)


def _split_box(box, rng, depth):
    offset, shape = box
    dims = [d for d in range(len(shape)) if shape[d] > 1]
    if depth == 0 or not dims or rng.random() < 0.2:
        return [box]
    d = rng.choice(dims)
    cut = rng.randrange(1, shape[d])
    low = (list(offset), list(shape))
    low[1][d] = cut
    high = (list(offset), list(shape))
    high[0][d] += cut
    high[1][d] -= cut
    return _split_box(low, rng, depth - 1) + _split_box(high, rng, depth - 1)


def _random_reshards(rank, world, port, seed, count):
    import random

    dist = init_moodist(rank, world, port)
    import moodist_b200 as moodist

    pg = moodist.get_backend(device="cpu")
    rng = random.Random(seed)  # the same on every rank: all of them know every rank's boxes
    for case in range(count):
        nd = rng.randint(1, 4)
        shape = [rng.randint(1, (200, 40, 12, 7)[nd - 1]) for _ in range(nd)]
        dtype = rng.choice([torch.float32, torch.bfloat16, torch.int64, torch.uint8, torch.float64])
        full = torch.randint(0, 200, shape, generator=torch.Generator().manual_seed(seed * 1000 + case)).to(dtype)
        # inputs: the tensor cut into up to 16 boxes dealt to random ranks, some of them held by a second rank too;
        # outputs: up to three arbitrary boxes per rank, which straddle the inputs as they please
        pieces = _split_box(([0] * nd, shape), rng, rng.randint(0, 4))
        held = {r: [] for r in range(world)}
        for piece in pieces:
            held[rng.randrange(world)].append(piece)
            second = rng.randrange(world)
            if rng.random() < 0.2 and piece not in held[second]:
                held[second].append(piece)
        wanted = {r: [] for r in range(world)}
        for r in range(world):
            for _ in range(rng.randint(0, 3)):
                offset = [rng.randrange(s) for s in shape]
                wanted[r].append((offset, [rng.randint(1, s - o) for s, o in zip(shape, offset)]))

        def boxes(items):
            return [{"offset": list(o), "shape": list(s)} for o, s in items] or None

        op = moodist.compile_op(pg, shape=tuple(shape), dtype=dtype, inputs=boxes(held[rank]), outputs=boxes(wanted[rank]))
        for it in range(2):
            src = full + it if dtype != torch.uint8 else full

            def cut(box):
                return src[tuple(slice(o, o + s) for o, s in zip(*box))].contiguous()

            outs = [torch.full(box[1], 99, dtype=dtype) for box in wanted[rank]]
            op([cut(box) for box in held[rank]], outs).wait()
            for out, box in zip(outs, wanted[rank]):
                assert torch.equal(out, cut(box)), (case, it, shape, box, held, wanted)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("direct", ["1", "0"])
def test_compile_op_random_boxes_in_one_to_four_dimensions(direct):
    run_ranks(_random_reshards, 3, 7 + int(direct), 40, timeout=240, env={"MOODIST_DIRECT_CPU": direct})
