"""bf16 GEMMs on the hand-written tcgen05 kernel, with autograd.

``linear(x, w)`` is ``x @ w.T`` (the ``torch.nn.functional.linear`` contract without bias) where all
three GEMMs of a training step — output, input gradient, weight gradient — run on the sm_100a kernel
in ``csrc/kernels/gemm_tcgen05.cuh``: the backward passes use its MN-major operand modes so no tensor is
transposed in memory.  There is no fallback: on a CUDA device the extension must be present.
"""

from __future__ import annotations

import torch

from .._core import _C

_launches = 0


def gemm_launches() -> int:
    """Number of tcgen05 GEMM kernels launched by this process so far."""
    return _launches


def gemm(a, b, trans_a=False, trans_b=False, out=None, out_fp32=False, epilogue=0):
    """``op(a) @ op(b).T`` in bf16 with fp32 accumulation.

    ``a`` is ``[M, K]`` (or ``[K, M]`` with ``trans_a``), ``b`` is ``[N, K]`` (or ``[K, N]`` with
    ``trans_b``); rows must be contiguous.  ``epilogue=1`` applies SiLU to the result.
    """
    global _launches
    _launches += 1
    return _C.gemm(a, b, trans_a, trans_b, out, out_fp32, epilogue)


def _rows_ok(t: torch.Tensor) -> bool:
    return t.stride(-1) == 1 and (t.stride(0) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        # a sharded engine may hand the weight a slot in its flat gradient buffer: the weight-gradient
        # GEMM then writes there directly and autograd sees no gradient for the weight
        ctx.grad_slot = getattr(w, "_mb_grad_slot", None)
        x2 = x.reshape(-1, x.shape[-1])
        if not _rows_ok(x2):
            x2 = x2.contiguous()
        # allocate the result in its final shape: the caller may update it in place (rotary embedding,
        # cross-entropy gradient), which autograd forbids on a view made inside a custom Function
        y = torch.empty(*x.shape[:-1], w.shape[0], device=x.device, dtype=torch.bfloat16)
        gemm(x2, w, out=y.view(-1, w.shape[0]))
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not _rows_ok(gy2):
            gy2 = gy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        if not _rows_ok(x2):
            x2 = x2.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            # dx[T, K] = dy[T, N] @ w[N, K]: w is the MN-major "B" operand
            gx = gemm(gy2, w, trans_b=True).view(x.shape)
        if ctx.needs_input_grad[1]:
            # dw[N, K] = dy[T, N]^T @ x[T, K]: both operands MN-major
            slot = ctx.grad_slot
            if slot is not None and not slot.written and gy2.is_cuda:
                gemm(gy2, x2, trans_a=True, trans_b=True, out=slot.view)
                slot.written = True
            else:
                gw = gemm(gy2, x2, trans_a=True, trans_b=True)
        return gx, gw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for bf16 CUDA tensors; differentiable in both arguments."""
    return _Linear.apply(x, w)


class Linear(torch.nn.Module):
    """Bias-free linear layer whose forward and backward GEMMs run on the tcgen05 kernel.

    A sharding engine may take the weight over (``parallel.regather``): it then leaves a handle on the module
    and the layer's matmuls, the gathering of the weight and its gradient all go through that handle.
    ``fuse_gather=True`` marks a layer whose weight all-gather such an engine should fuse into the GEMM.
    """

    _mb_regather_kind = "linear"

    def __init__(self, in_features: int, out_features: int, device=None, dtype=torch.bfloat16, fuse_gather=False):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self._mb_fuse_gather = bool(fuse_gather)
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.weight._mb_linear_weight = True  # lets a sharded engine route the weight gradient (see _Linear)

    def reset_parameters(self, std: float = 0.02) -> None:
        torch.nn.init.normal_(self.weight, mean=0.0, std=std)

    def forward(self, x):
        h = self.__dict__.get("_mb_handle")
        if h is not None:
            return h.linear(x)
        w = self.weight
        if w.is_cuda and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
            return linear(x, w)
        return torch.nn.functional.linear(x, w)
