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


def _adopt(holder, key, value, what):
    """Record the global shape / dtype the first DTensor brings; later ones must agree."""
    if holder.get(key) is None:
        holder[key] = value
    elif holder[key] != value:
        raise ValueError(f"compile_op: DTensors disagree on the global {what}: {holder[key]} here, {value} there")


def _normalise(specs, holder):
    if specs is None:
        return None
    out = []
    for x in specs:
        if _is_dtensor(x):
            _adopt(holder, "shape", tuple(x.shape), "shape")
            _adopt(holder, "dtype", x.dtype, "dtype")
            out.append(_shard_box(x))
        else:
            out.append(x)
    return out


def _int_list(box, field, ndim, where):
    if field not in box:
        raise ValueError(f"compile_op: {where} has no '{field}' entry")
    values = box[field]
    if not isinstance(values, (tuple, list)):
        raise TypeError(f"compile_op: '{field}' of {where} is a {type(values).__name__}; a list or tuple of ints is needed")
    if len(values) != ndim:
        raise ValueError(f"compile_op: '{field}' of {where} has {len(values)} entries for a {ndim}-d tensor")
    for i, v in enumerate(values):
        if not isinstance(v, int) or isinstance(v, bool):
            raise TypeError(f"compile_op: {field}[{i}] of {where} is a {type(v).__name__}, not an int")
    return tuple(values)


def _check(specs, ndim, side):
    if not isinstance(specs, (tuple, list)):
        raise TypeError(f"compile_op: {side} is a {type(specs).__name__}; pass a list of boxes (or None)")
    boxes = []
    for index, box in enumerate(specs):
        where = f"{side}[{index}]"
        if not isinstance(box, dict):
            raise TypeError(f"compile_op: {where} is a {type(box).__name__}; a box is a dict with 'offset' and 'shape'")
        boxes.append((_int_list(box, "offset", ndim, where), _int_list(box, "shape", ndim, where)))
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
    raise RuntimeError(f"compile_op: {type(group).__name__} is not a moodist process group")


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
    if shape is None or dtype is None:
        missing = "shape" if shape is None else "dtype"
        raise ValueError(f"compile_op: give the global {missing}, or pass DTensors that carry it")
    if not isinstance(dtype, torch.dtype):
        raise TypeError(f"compile_op: dtype is a {type(dtype).__name__}, not a torch.dtype")
    shape = tuple(shape)
    for i, x in enumerate(shape):
        if not isinstance(x, int) or isinstance(x, bool):
            raise TypeError(f"compile_op: shape[{i}] is a {type(x).__name__}, not an int")
    if inputs is not None:
        inputs = _check(inputs, len(shape), "inputs")
    if outputs is not None:
        outputs = _check(outputs, len(shape), "outputs")

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
            raise ValueError(f"compile_op: rank {source_rank} describes a {tuple(nshape)} tensor, this rank a {shape} one")
        if ndtype != str(dtype):
            raise ValueError(f"compile_op: rank {source_rank} describes {ndtype} data, this rank {dtype}")
        for o, s in ninput or ():
            all_inputs.append((source_rank, list(o), list(s)))
        for o, s in noutput or ():
            all_outputs.append((source_rank, list(o), list(s)))
    pg.barrier().wait()
    # every rank must build the plan from the same list
    all_inputs.sort(key=lambda t: t[0])
    all_outputs.sort(key=lambda t: t[0])
    return pg.compile_op_full(list(shape), dtype, all_inputs, all_outputs)
