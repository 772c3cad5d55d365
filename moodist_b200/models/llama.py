"""Llama-3-shaped decoder used by the FSDP benchmark and the smoke test.

The reference library has no model code (it is a communication backend); its FSDP2 benchmark target is
a Llama-3-8B-shaped network: 32 layers, d=4096, 32 heads / 8 KV heads, SwiGLU FFN 14336, vocabulary
128256, RoPE theta 500000, RMSNorm.  Every projection is a ``moodist_b200.ops.gemm.Linear`` so the
matrix products of forward and backward run on the tcgen05 kernel; rotary embedding, SwiGLU and the
cross-entropy are the single-pass kernels of ``moodist_b200.ops.train``; attention uses torch's fused SDPA
(cuDNN's sm_100 flash kernels on a B200).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..ops.gemm import Linear
from ..ops.train import cross_entropy, rms_norm, rope_qkv_, swiglu


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    max_seq_len: int = 8192

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(vocab_size=1024, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512, max_seq_len=256)

    def num_params(self) -> int:
        hd = self.dim // self.n_heads
        attn = self.dim * (self.n_heads * hd) + 2 * self.dim * (self.n_kv_heads * hd) + (self.n_heads * hd) * self.dim
        mlp = 3 * self.dim * self.ffn_dim
        return self.n_layers * (attn + mlp + 2 * self.dim) + 2 * self.vocab_size * self.dim + self.dim


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return rms_norm(x, self.weight, self.eps)


def rope_tables(head_dim: int, seq_len: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    freqs = torch.outer(t, inv)
    return freqs.cos(), freqs.sin()


class RopeTables:
    """fp32 cos / sin tables handed to the blocks as one opaque object, so that wrappers which cast tensor
    arguments to the compute dtype (FSDP2 mixed precision) leave their precision alone."""

    __slots__ = ("cos", "sin")

    def __init__(self, cos: torch.Tensor, sin: torch.Tensor):
        self.cos, self.sin = cos, sin


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x: [B, S, H, D]; rotate pairs (even, odd halves layout)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c = cos[None, : x.shape[1], None, :]
    s = sin[None, : x.shape[1], None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None):
        super().__init__()
        self.n_heads, self.n_kv = cfg.n_heads, cfg.n_kv_heads
        self.hd = cfg.dim // cfg.n_heads
        # fused QKV projection: one GEMM whose gathered weight arrives through the all-gather
        self.wqkv = Linear(cfg.dim, (cfg.n_heads + 2 * cfg.n_kv_heads) * self.hd, device=device, fuse_gather=True)
        self.wo = Linear(cfg.n_heads * self.hd, cfg.dim, device=device)

    def forward(self, x, rope: RopeTables):
        cos, sin = rope.cos, rope.sin
        B, S, _ = x.shape
        # q and k heads are rotated in place inside the projection's output (nothing else reads it)
        qkv = rope_qkv_(self.wqkv(x), cos, sin, self.n_heads + self.n_kv, self.hd)
        q, k, v = qkv.split([self.n_heads * self.hd, self.n_kv * self.hd, self.n_kv * self.hd], dim=-1)
        q = q.view(B, S, self.n_heads, self.hd).transpose(1, 2)
        k = k.view(B, S, self.n_kv, self.hd).transpose(1, 2)
        v = v.view(B, S, self.n_kv, self.hd).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.wo(o.transpose(1, 2).reshape(B, S, self.n_heads * self.hd))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None):
        super().__init__()
        # gate and up projections share one GEMM (the "up" GEMM the all-gather is fused into)
        self.w13 = Linear(cfg.dim, 2 * cfg.ffn_dim, device=device, fuse_gather=True)
        self.w2 = Linear(cfg.ffn_dim, cfg.dim, device=device)

    def forward(self, x):
        return self.w2(swiglu(self.w13(x)))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device)
        self.attn = Attention(cfg, device=device)
        self.mlp_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device)
        self.mlp = MLP(cfg, device=device)

    def forward(self, x, rope: RopeTables):
        x = x + self.attn(self.attn_norm(x), rope)
        return x + self.mlp(self.mlp_norm(x))


class Embedding(nn.Embedding):
    """Token embedding whose table a sharding engine may take over (it then leaves a handle on the module)."""

    _mb_regather_kind = "embedding"

    def forward(self, tokens):
        h = self.__dict__.get("_mb_handle")
        if h is not None:
            return h.embedding(tokens)
        return super().forward(tokens)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed = Embedding(cfg.vocab_size, cfg.dim, device=device, dtype=torch.bfloat16)
        self.layers = nn.ModuleList([Block(cfg, device=device) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device)
        self.lm_head = Linear(cfg.dim, cfg.vocab_size, device=device)
        self._rope = None

    def init_weights(self, seed: int = 0) -> None:
        g = torch.Generator(device=self.embed.weight.device).manual_seed(seed)
        for p in self.parameters():
            if p.dim() >= 2:
                with torch.no_grad():
                    p.normal_(0.0, 0.02, generator=g)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        S = tokens.shape[1]
        if self._rope is None or self._rope[0].shape[0] < S or self._rope[0].device != tokens.device:
            self._rope = rope_tables(self.cfg.dim // self.cfg.n_heads, max(S, 16), self.cfg.rope_theta, tokens.device)
        rope = RopeTables(*self._rope)
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x, rope)
        return self.lm_head(self.norm(x))


def loss_fn(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean token cross-entropy; on CUDA the backward overwrites ``logits`` with its gradient."""
    return cross_entropy(logits, targets)
