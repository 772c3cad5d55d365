"""Memory-bound pieces of the training step as single-pass sm_100a kernels, with autograd.

``rope_qkv_``     rotary embedding applied in place to the q and k heads of the fused QKV activations
``swiglu``        ``silu(gate) * up`` on the fused gate/up activations; the backward is one kernel too
``cross_entropy`` mean token cross-entropy over bf16 logits; the backward overwrites the logits with their
                  gradient, so no fp32 copy of the ``[tokens, vocab]`` matrix is ever made
``adamw_``        AdamW over a flat bf16 parameter shard with bf16 moments (gradient fp32 or bf16)
``rms_norm``      RMSNorm over the last dimension; the backward produces dx and dw in one pass over dy and x

On CUDA tensors these always run the kernels of ``csrc/kernels/train_ops.cu``.  CPU tensors take plain
PyTorch arithmetic so the sharded engine's host-side logic can be exercised on ``gloo`` ranks.
The reference library is a communication backend and has no counterpart of these ops.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .._core import _C

_launches = 0


def train_op_launches() -> int:
    """Number of kernels launched by this module so far in this process."""
    return _launches


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def _rope_reference(x2, cos, sin, seq, n_heads, head_dim, inverse):
    t = x2.shape[0]
    v = x2[:, : n_heads * head_dim].reshape(t, n_heads, head_dim).float()
    half = head_dim // 2
    pos = torch.arange(t, device=x2.device) % seq
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :] * (-1.0 if inverse else 1.0)
    a, b = v[..., :half], v[..., half:]
    out = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    x2[:, : n_heads * head_dim] = out.reshape(t, n_heads * head_dim).to(x2.dtype)


def _rope_apply(x2, cos, sin, seq, n_heads, head_dim, inverse):
    if x2.is_cuda:
        _count()
        _C.rope_(x2, cos, sin, seq, n_heads, head_dim, inverse)
    else:
        _rope_reference(x2, cos, sin, seq, n_heads, head_dim, inverse)


class _RopeQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, seq, n_heads, head_dim):
        ctx.save_for_backward(cos, sin)
        ctx.args = (seq, n_heads, head_dim)
        x2 = qkv.view(-1, qkv.shape[-1])
        _rope_apply(x2, cos, sin, seq, n_heads, head_dim, False)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        seq, n_heads, head_dim = ctx.args
        g = g.contiguous() if not g.is_contiguous() else g
        g2 = g.view(-1, g.shape[-1])
        # the incoming gradient is a fresh buffer (assembled from dq, dk, dv): rotate it in place
        _rope_apply(g2, cos, sin, seq, n_heads, head_dim, True)
        return g, None, None, None, None, None


def rope_qkv_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, head_dim: int) -> torch.Tensor:
    """Rotate the first ``n_rot_heads`` heads (q then k) of ``qkv[B, S, (H + 2 KV) * head_dim]`` in place.

    Pairs are ``(j, j + head_dim/2)``; ``cos``/``sin`` are fp32 ``[>= S, head_dim/2]``.  ``qkv`` must be a
    tensor nobody else needs unrotated (the output of the QKV projection).
    """
    return _RopeQKV.apply(qkv, cos, sin, qkv.shape[-2], n_rot_heads, head_dim)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        gu2 = gu.reshape(-1, gu.shape[-1])
        if gu2.is_cuda:
            _count()
            out = _C.swiglu_fwd(gu2)
        else:
            g, u = gu2.float().chunk(2, dim=-1)
            out = (F.silu(g) * u).to(gu.dtype)
        return out.view(*gu.shape[:-1], gu.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        gu2 = gu.reshape(-1, gu.shape[-1])
        d2 = dout.reshape(-1, dout.shape[-1])
        if gu2.is_cuda:
            if d2.stride(-1) != 1 or (d2.stride(0) * 2) % 16:
                d2 = d2.contiguous()
            _count()
            dgu = _C.swiglu_bwd(gu2, d2)
        else:
            g, u = gu2.float().chunk(2, dim=-1)
            sig = torch.sigmoid(g)
            sl = g * sig
            d = d2.float()
            dgu = torch.cat([d * u * (sig + sl * (1 - sig)), d * sl], dim=-1).to(gu.dtype)
        return dgu.view(gu.shape)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gu[..., :F]) * gu[..., F:]`` for the fused gate/up projection output."""
    return _SwiGLU.apply(gu)


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index):
        l2 = logits.view(-1, logits.shape[-1])
        t = targets.reshape(-1).contiguous()
        # mean over the rows that are not ignored (kept on the device: no synchronisation)
        count = (t != ignore_index).sum().clamp(min=1).float()
        _count()
        rows, lse = _C.cross_entropy_fwd(l2, t, ignore_index)
        ctx.save_for_backward(l2, t, lse, count)
        ctx.ignore_index = ignore_index
        ctx.shape = logits.shape
        return rows.sum() / count

    @staticmethod
    def backward(ctx, g):
        l2, t, lse, count = ctx.saved_tensors
        gs = g.reshape(1).float() / count
        _count()
        _C.cross_entropy_bwd_(l2, t, lse, gs, 1.0, ctx.ignore_index)
        return l2.view(ctx.shape), None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy of bf16 ``logits[..., V]`` against int64 ``targets``.

    On CUDA the backward pass writes the gradient over ``logits`` (the output of the last projection,
    which nothing else reads); the returned loss is an fp32 scalar.
    """
    if not logits.is_cuda:
        return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=ignore_index)
    if not logits.is_contiguous():
        logits = logits.contiguous()
    return _CrossEntropy.apply(logits, targets, ignore_index)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1 or (x2.stride(0) * 2) % 16:
            x2 = x2.contiguous()
        _count()
        y, rstd = _C.rmsnorm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, w, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        d2 = dy.reshape(-1, dy.shape[-1])
        if d2.stride(-1) != 1 or (d2.stride(0) * 2) % 16:
            d2 = d2.contiguous()
        _count(2)
        dx, dw = _C.rmsnorm_bwd(x2, w, d2, rstd)
        return dx.view(dy.shape), dw, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2, -1) + eps) * weight``; bf16 CUDA tensors whose last dimension is a multiple of 8
    (up to 8192) run the single-pass kernels, anything else ``torch.nn.functional.rms_norm``."""
    d = x.shape[-1]
    if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and d % 8 == 0
            and d <= _C.rmsnorm_max_dim() and weight.is_contiguous()):
        return _RMSNorm.apply(x, weight, eps)
    return F.rms_norm(x, (d,), weight, eps)


def adamw_(p, g, m, v, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, step: int = 1,
           grad_scale: float = 1.0) -> None:
    """One AdamW update of the flat bf16 tensor ``p`` in place (decoupled decay, bias-corrected).

    ``g`` is the gradient (fp32 or bf16, multiplied by ``grad_scale`` first), ``m``/``v`` the bf16 moments.
    """
    b1, b2 = betas
    if p.is_cuda:
        _count()
        _C.adamw_(p, g, m, v, lr, b1, b2, eps, weight_decay, step, grad_scale)
        return
    gr = g.float() * grad_scale
    mf = m.float().mul_(b1).add_(gr, alpha=1 - b1)
    vf = v.float().mul_(b2).addcmul_(gr, gr, value=1 - b2)
    bc1 = 1 - b1**step
    bc2 = 1 - b2**step
    denom = vf.sqrt() / (bc2**0.5) + eps
    pf = p.float() * (1 - lr * weight_decay) - (lr / bc1) * mf / denom
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)


def adamw_master_(p, master, g, m, v, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                  step: int = 1) -> None:
    """AdamW on an fp32 master copy with fp32 moments; ``p`` (any float dtype, usually bf16) receives the rounded
    result.  The arithmetic mixed-precision FSDP keeps per shard: ``master``, ``m`` and ``v`` are fp32 tensors of
    ``p``'s shape, ``g`` the gradient in fp32 or bf16.  Plain PyTorch ops on whatever device the tensors live on
    (several passes over the shard; the single-pass kernel is ``adamw_``, which keeps bf16 state)."""
    b1, b2 = betas
    gr = g if g.dtype == torch.float32 else g.float()
    m.mul_(b1).add_(gr, alpha=1 - b1)
    v.mul_(b2).addcmul_(gr, gr, value=1 - b2)
    bc1 = 1 - b1**step
    bc2 = 1 - b2**step
    denom = v.sqrt().div_(bc2**0.5).add_(eps)
    master.mul_(1 - lr * weight_decay).addcdiv_(m, denom, value=-lr / bc1)
    p.copy_(master)
