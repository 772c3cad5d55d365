"""Sharded data-parallel training of the Llama-shaped decoder over the moodist backend.

``ShardedTrainer`` is the public training entry point: it builds the model on the local GPU, shards
every transformer block with torch's FSDP2 ``fully_shard`` on a process group whose collectives are this
library's sm_100a kernels (per-layer all-gather of bf16 parameters, reduce-scatter of gradients with
fp32 accumulation and the 1/world average folded into the kernel), and exposes ``step(tokens)``, which
takes a pinned host batch and returns the loss as a Python float.

The reference ships no trainer; FSDP2 over its process group is how it is benchmarked, so the same
construction is used here (``fully_shard`` needs all_gather_into_tensor, reduce_scatter_tensor,
all_reduce, broadcast and barrier from the backend).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

from ..models.llama import Llama, LlamaConfig, loss_fn


class ShardedTrainer:
    """FSDP2 training of a Llama-shaped decoder with bf16 parameters and fp32 gradient reduction."""

    def __init__(
        self,
        cfg: LlamaConfig,
        group: dist.ProcessGroup | None = None,
        lr: float = 1e-4,
        seed: int = 0,
        reshard_after_forward: bool = True,
    ):
        if not torch.cuda.is_available():
            raise RuntimeError("ShardedTrainer needs a CUDA device")
        self.cfg = cfg
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        torch.manual_seed(seed)
        self.model = Llama(cfg, device=self.device)
        self.model.init_weights(seed)
        ranks = dist.get_process_group_ranks(self.group)
        mesh = DeviceMesh.from_group(self.group, "cuda", mesh=torch.tensor(ranks), mesh_dim_names=("dp",))
        policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for layer in self.model.layers:
            fully_shard(layer, mesh=mesh, mp_policy=policy, reshard_after_forward=reshard_after_forward)
        fully_shard(self.model, mesh=mesh, mp_policy=policy, reshard_after_forward=reshard_after_forward)
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
        self._tok_dev = None

    def step_on_device(self, tokens: torch.Tensor) -> torch.Tensor:
        """One optimizer step on a batch that already lives on the GPU; returns the loss tensor."""
        inp, tgt = tokens[:, :-1], tokens[:, 1:]
        logits = self.model(inp)
        loss = loss_fn(logits, tgt)
        loss.backward()
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss

    def step(self, tokens_host: torch.Tensor) -> float:
        """One optimizer step from a (pinned) host batch of token ids ``[B, S+1]``; returns the loss."""
        if self._tok_dev is None or self._tok_dev.shape != tokens_host.shape:
            self._tok_dev = torch.empty(tokens_host.shape, dtype=tokens_host.dtype, device=self.device)
        self._tok_dev.copy_(tokens_host, non_blocking=True)
        return float(self.step_on_device(self._tok_dev).item())
