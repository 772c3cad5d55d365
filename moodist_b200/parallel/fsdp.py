"""Sharded data-parallel training of the Llama-shaped decoder over the moodist backend.

``ShardedTrainer`` is the public training entry point: it builds the model on the local GPU, shards it
over a process group whose collectives are this library's sm_100a kernels, and exposes ``step(tokens)``,
which takes a pinned host batch and returns the loss as a Python float.  Two engines:

``engine="native"`` (default) with ``schedule="regather"`` (default)
    ``moodist_b200.parallel.regather.RegatherEngine``: the FSDP2 schedule on this library's own kernels.
    Parameters are sharded by rows at rest; a block's weights are gathered for its forward and again for its
    backward.  The gathers of the QKV and gate/up weights happen inside their GEMM kernels
    (``ops.fused.ag_gemm``), the others one block ahead on a side stream; weight gradients leave through a
    reduce-scatter (bf16 on the wire, fp32 sum) per weight as soon as the GEMM that made them is done, and
    AdamW updates this rank's rows.
``engine="native"`` with ``schedule="resident"``  ``moodist_b200.parallel.sharded.ShardedEngine``: gathered
    parameters stay resident (only possible while the whole model fits one GPU), gradients are
    reduce-scattered from bf16 with fp32 accumulation, AdamW runs on the flat shard and the updated shard
    is all-gathered in place, all per unit on a side stream under the rest of the backward pass.
``engine="fsdp2"``  torch's ``fully_shard`` per transformer block (bf16 parameters, fp32 reduce), the
    construction the reference is benchmarked under; needs all_gather_into_tensor,
    reduce_scatter_tensor, all_reduce, broadcast and barrier from the backend.

The reference ships no trainer of its own.
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
        engine: str = "native",
        symmetric_memory: bool = True,
        schedule: str = "regather",
        fused: bool = True,
        copy_engine: bool | None = None,
        master_weights: bool = False,
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
        self.engine = None
        self.opt = None
        self.schedule = schedule if engine == "native" else "fsdp2"
        # The re-gather schedule keeps the side stream busy through forward and backward. Measured on 8 GPUs, its
        # plain gathers and reduce-scatters cost the concurrent GEMMs less when the bytes move with DMA copies
        # between one-warp flag kernels (448.5 ms per step) than with SM copy kernels (457.1 ms), so that is the
        # default for it; `copy_engine=False` keeps the SM kernels, `True` forces DMA for any schedule.
        if copy_engine is None:
            copy_engine = engine == "native" and schedule == "regather"
        self.copy_engine = False
        if copy_engine and self.world > 1 and dist.get_backend(self.group) == "moodist":
            from ..backend import get_backend

            get_backend(self.group).set_prefer_kernel_less(True)
            self.copy_engine = True
        if engine == "native":
            m = self.model
            units = [("embed", [m.embed])]
            units += [(f"layers.{i}", [layer]) for i, layer in enumerate(m.layers)]
            units += [("head", [m.norm, m.lm_head])]
            if schedule == "regather":
                from .regather import RegatherEngine

                names = {id(p): n for n, p in m.named_parameters()}
                self.engine = RegatherEngine(units, group=self.group, lr=lr, betas=(0.9, 0.95), weight_decay=0.1,
                                             fused=fused, symmetric_memory=symmetric_memory, param_names=names,
                                             master_weights=master_weights)
            elif schedule == "resident":
                from .sharded import ShardedEngine

                self.engine = ShardedEngine(units, group=self.group, lr=lr, betas=(0.9, 0.95), weight_decay=0.1,
                                            symmetric_memory=symmetric_memory)
            else:
                raise ValueError(f"unknown schedule {schedule!r} (regather or resident)")
        elif engine == "fsdp2":
            ranks = dist.get_process_group_ranks(self.group)
            mesh = DeviceMesh.from_group(self.group, "cuda", mesh=torch.tensor(ranks), mesh_dim_names=("dp",))
            policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
            for layer in self.model.layers:
                fully_shard(layer, mesh=mesh, mp_policy=policy, reshard_after_forward=reshard_after_forward)
            fully_shard(self.model, mesh=mesh, mp_policy=policy, reshard_after_forward=reshard_after_forward)
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1,
                                         fused=True)
        else:
            raise ValueError(f"unknown engine {engine!r} (native or fsdp2)")
        self._tok_dev = None

    def step_on_device(self, tokens: torch.Tensor) -> torch.Tensor:
        """One optimizer step on a batch that already lives on the GPU; returns the loss tensor."""
        inp, tgt = tokens[:, :-1], tokens[:, 1:]
        logits = self.model(inp)
        loss = loss_fn(logits, tgt)
        loss.backward()
        if self.engine is not None:
            self.engine.finish_step()
        else:
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
        return loss

    def step(self, tokens_host: torch.Tensor) -> float:
        """One optimizer step from a (pinned) host batch of token ids ``[B, S+1]``; returns the loss."""
        if self._tok_dev is None or self._tok_dev.shape != tokens_host.shape:
            self._tok_dev = torch.empty(tokens_host.shape, dtype=tokens_host.dtype, device=self.device)
        self._tok_dev.copy_(tokens_host, non_blocking=True)
        return float(self.step_on_device(self._tok_dev).item())
