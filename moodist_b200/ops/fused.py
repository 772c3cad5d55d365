"""Fused collective GEMMs: all-gather -> GEMM and GEMM -> reduce-scatter in one sm_100a kernel each.

``ag_gemm`` pushes this rank's shard to every peer's staging area from a few copy CTAs while the other
CTAs of the same grid run the tcgen05 GEMM, consuming shards in the order they land.  ``gemm_rs`` lets the
GEMM epilogue write bf16 partial tiles straight into the owning rank's memory and reduces them there in
fp32.  Both are what tensor-/sequence-parallel blocks and FSDP layers do around their matmuls; the
unfused equivalents are ``dist.all_gather_into_tensor`` + ``gemm`` and ``gemm`` + ``dist.reduce_scatter_tensor``.
"""

from __future__ import annotations

import torch

from .._core import _C

_launches = 0


def fused_launches() -> int:
    return _launches


def ag_gemm(group, shard, other, gather_weight=False, out_fp32=False, epilogue=0, comm_ctas=0, out=None):
    """``all_gather(shard) @ other.T`` (``gather_weight=False``) or ``other @ all_gather(shard).T``.

    Returns ``(y, gathered)``; ``gathered`` aliases the group's staging area and is valid until the
    collective after next on this group.  ``out`` (contiguous ``[M, N]``) receives ``y`` when given.
    """
    global _launches
    _launches += 1
    return _C.ag_gemm(group, shard, other, gather_weight, out_fp32, epilogue, comm_ctas, out)


def gemm_rs(group, a, b, trans_b=False, out_fp32=False, scale=1.0):
    """``reduce_scatter(a @ b.T)`` over rows: rank r gets rows ``[r*M/world, (r+1)*M/world)`` of the sum."""
    global _launches
    _launches += 1
    return _C.gemm_rs(group, a, b, trans_b, out_fp32, scale)
