"""``compile_op``: plan an arbitrary redistribution of an N-d tensor once, run it many times.

Every rank says which boxes of a global tensor it holds (``inputs``) and which boxes it wants
(``outputs``) — as ``{'offset': [...], 'shape': [...]}`` dicts or as DTensors — and gets back a callable
``op(input_tensors, output_tensors)``.  all-gather, scatter, gather, broadcast, row-sharded ->
column-sharded, 2-D block -> 1-D row layouts are all instances.  On CUDA tensors the plan runs as one
sm_100a gather/scatter kernel over peer memory; on CPU tensors the host engine pulls the pieces.

API and metadata exchange follow the reference (``py/moodist/compile.py:16-264``): specs are normalised,
exchanged between all ranks through a named multicast Queue, validated, then handed to
``group.compile_op_full``.  The call is collective.
"""

from __future__ import annotations

import weakref

import torch

from .queue import Queue

_queues: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()


def _is_dtensor(x) -> bool:
    return hasattr(x, "placements") and hasattr(x, "device_mesh") and hasattr(x, "to_local")


def _shard_box(dtensor) -> dict:
    """Offset and local shape of this rank's shard, using torch's ceil-division chunking of ``Shard``."""
    from torch.distributed.tensor import Shard

    mesh = dtensor.device_mesh
    shape = list(dtensor.shape)
    offset = [0] * len(shape)
    local = list(shape)
    coord = mesh.get_coordinate()
    if coord is None:  # this rank is not part of the mesh
        return {"offset": offset, "shape": [0] * len(shape)}
    for mesh_dim, placement in enumerate(dtensor.placements):
        if not isinstance(placement, Shard):
            continue
        d = placement.dim
        # a dimension sharded over several mesh dims is split again inside the outer shard
        size, start = local[d], offset[d]
        parts = mesh.size(mesh_dim)
        chunk = -(-size // parts)
        begin = min(size, chunk * coord[mesh_dim])
        end = min(size, begin + chunk)
        offset[d] = start + begin
        local[d] = end - begin
    return {"offset": offset, "shape": local}


def _normalise(specs, holder):
    if specs is None:
        return None
    out = []
    for x in specs:
        if _is_dtensor(x):
            shape, dtype = tuple(x.shape), x.dtype
            if holder.get("shape") is None:
                holder["shape"] = shape
            elif tuple(holder["shape"]) != shape:
                raise ValueError(f"All DTensors must have the same global shape, got {holder['shape']} and {shape}")
            if holder.get("dtype") is None:
                holder["dtype"] = dtype
            elif holder["dtype"] != dtype:
                raise ValueError(f"All DTensors must have the same dtype, got {holder['dtype']} and {dtype}")
            out.append(_shard_box(x))
        else:
            out.append(x)
    return out


def _check(specs, ndim):
    if not isinstance(specs, (tuple, list)):
        raise TypeError(f"inputs/outputs must be a tuple or list, got {type(specs).__name__}")
    boxes = []
    for x in specs:
        if not isinstance(x, dict):
            raise TypeError(f"each input/output spec must be a dict, got {type(x).__name__}")
        for n in ("offset", "shape"):
            if n not in x:
                raise ValueError(f"'{n}' is missing for an input or output")
            v = x[n]
            if not isinstance(v, (tuple, list)):
                raise TypeError(f"'{n}' must be a tuple or list, got {type(v).__name__}")
            if len(v) != ndim:
                raise ValueError(f"expected '{n}' with {ndim} dimensions, but got {len(v)}")
            for i, z in enumerate(v):
                if not isinstance(z, int):
                    raise TypeError(f"{n}[{i}] must be an int, got {type(z).__name__}")
        boxes.append((tuple(x["offset"]), tuple(x["shape"])))
    return tuple(boxes)


def _backend_of(group):
    if hasattr(group, "compile_op_full"):
        return group
    if hasattr(group, "_get_backend"):
        for dev in ("cpu", "cuda"):
            try:
                b = group._get_backend(torch.device(dev))
            except RuntimeError:
                continue
            if hasattr(b, "compile_op_full"):
                return b
    raise RuntimeError(f"moodist.compile_op needs a moodist process group, got {type(group)}")


def compile_op(group, shape=None, dtype=None, inputs=None, outputs=None):
    """Compile a redistribution of a global ``shape``/``dtype`` tensor. Collective over ``group``.

    ``inputs`` / ``outputs``: lists of ``{'offset', 'shape'}`` dicts in global coordinates, or DTensors
    (shape and dtype are then taken from them); ``None`` when this rank contributes / receives nothing.
    Returns ``op`` with ``op(input_tensors, output_tensors) -> future``; tensors are contiguous local
    buffers of the boxes' shapes, all CPU or all CUDA.
    """
    pg = _backend_of(group)
    holder = {"shape": tuple(shape) if shape is not None else None, "dtype": dtype}
    inputs = _normalise(inputs, holder)
    outputs = _normalise(outputs, holder)
    shape, dtype = holder["shape"], holder["dtype"]
    if shape is None:
        raise ValueError("shape must be provided or derivable from DTensors")
    if dtype is None:
        raise ValueError("dtype must be provided or derivable from DTensors")
    if not isinstance(dtype, torch.dtype):
        raise TypeError(f"dtype must be a torch.dtype, got {type(dtype).__name__}")
    shape = tuple(shape)
    for i, x in enumerate(shape):
        if not isinstance(x, int):
            raise TypeError(f"shape[{i}] must be an int, got {type(x).__name__}")
    if inputs is not None:
        inputs = _check(inputs, len(shape))
    if outputs is not None:
        outputs = _check(outputs, len(shape))

    queue = _queues.get(pg)
    if queue is None:
        queue = Queue(pg, range(pg.size()), name=pg.moodist_name() + ".{compile_collective_queue}")
        _queues[pg] = queue

    pg.barrier().wait()
    queue.put_object((pg.rank(), shape, str(dtype), inputs, outputs))
    all_inputs, all_outputs = [], []
    for _ in range(pg.size()):
        source_rank, nshape, ndtype, ninput, noutput = queue.get_object()
        if tuple(nshape) != shape:
            raise ValueError(f"moodist.compile_op: Ranks specified different shapes: {shape} vs {nshape}")
        if ndtype != str(dtype):
            raise ValueError(f"moodist.compile_op: Ranks specified different dtypes: {dtype} vs {ndtype}")
        for o, s in ninput or ():
            all_inputs.append((source_rank, list(o), list(s)))
        for o, s in noutput or ():
            all_outputs.append((source_rank, list(o), list(s)))
    pg.barrier().wait()
    # every rank must build the plan from the same list
    all_inputs.sort(key=lambda t: t[0])
    all_outputs.sort(key=lambda t: t[0])
    return pg.compile_op_full(list(shape), dtype, all_inputs, all_outputs)
