"""Fully sharded data-parallel engine sized for 180 GB of HBM per GPU.

The classic fully-sharded schedule re-gathers every layer's parameters twice per step (forward and
backward) and frees them in between, because it was designed for GPUs on which the full model does not
fit.  A B200 holds a whole 8-B-parameter model in bf16 (16 GB) several times over, so this engine keeps
one *gathered* flat bf16 buffer per unit (a unit = one transformer block, the embedding, or the head)
resident all the time and shards only what is worth sharding: the optimizer state, the optimizer
arithmetic and the gradient reduction.  Per unit and per step it runs, on a side stream, as soon as the
unit's backward has finished:

    reduce-scatter(bf16 gradients -> fp32 average of this rank's slice)      (one kernel, cast fused)
    AdamW on the slice, written in place into the gathered buffer            (one kernel)
    all-gather in place of the updated slices                                (one kernel)

so both collectives and the optimizer of layer ``i`` overlap the backward pass of layers ``< i`` and
nothing is left for the forward pass to wait on except the tail of the first unit.  Parameters are
views into the gathered buffer, weight gradients are written by the GEMM straight into a flat gradient
buffer (no per-parameter copies, no concatenation).

With ``world_size == 1`` the collectives disappear and the engine is a flat-buffer optimizer.

The reference library ships no trainer (it is benchmarked under torch's FSDP2); this engine is the
B200-first replacement for that construction and runs over any ``torch.distributed`` backend, which is
how the NCCL comparison in ``bench.py`` is made.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..ops.train import adamw_

_ALIGN = 128  # elements; keeps every parameter view 256-byte aligned (TMA needs 16)


class GradSlot:
    """Where the weight-gradient GEMM of a ``Linear`` writes: a view into the unit's flat gradient buffer."""

    __slots__ = ("view", "written")

    def __init__(self, view: torch.Tensor):
        self.view = view
        self.written = False


@dataclass
class _Unit:
    name: str
    modules: list
    params: list = field(default_factory=list)
    offsets: list = field(default_factory=list)
    numel: int = 0          # padded, divisible by world * _ALIGN
    full: torch.Tensor | None = None       # gathered bf16 parameters [numel]
    grad: torch.Tensor | None = None       # flat bf16 gradients [numel]
    exp_avg: torch.Tensor | None = None    # [numel / world]
    exp_avg_sq: torch.Tensor | None = None
    ready: torch.cuda.Event | None = None  # parameters of the coming step are in place
    reduced: bool = True                   # this step's gradients were handed to the side stream


class _Boundary(torch.autograd.Function):
    """Identity on a unit's input; its backward runs after every other backward node of the unit."""

    @staticmethod
    def forward(ctx, x, engine, index):
        ctx.engine, ctx.index = engine, index
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.engine._unit_backward_done(ctx.index)
        return g, None, None


class ShardedEngine:
    """Shards optimizer state and gradient reduction of ``units`` over ``group``; see the module docstring.

    ``units`` is a list of ``(name, [modules])`` in forward execution order; every parameter of the model
    must belong to exactly one unit and be bf16 (CUDA) or any float dtype (CPU ranks used in tests).
    """

    def __init__(self, units, group=None, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 symmetric_memory=True, sync_init=True):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        self.units: list[_Unit] = []
        first = next(p for _, mods in units for m in mods for p in m.parameters())
        self.device = first.device
        self.cuda = self.device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._moodist = None
        if self.cuda and self.world > 1 and dist.get_backend(self.group) == "moodist":
            from ..backend import get_backend

            self._moodist = get_backend(self.group)
        self._symmetric = bool(symmetric_memory and self._moodist is not None)
        self._pool = None
        seen = set()
        for index, (name, mods) in enumerate(units):
            u = _Unit(name=name, modules=list(mods))
            for m in u.modules:
                for p in m.parameters():
                    if id(p) not in seen:
                        seen.add(id(p))
                        u.params.append(p)
            self._build_unit(u, sync_init)
            self.units.append(u)
            u.modules[0].register_forward_pre_hook(self._make_pre_hook(index), with_kwargs=True)

    # ---- construction ----------------------------------------------------------------------------
    def _alloc(self, numel, dtype, symmetric=False):
        if symmetric and self._symmetric:
            # peers read (and NVLS addresses) the gathered parameters in place: no staging copy per all-gather
            if self._pool is None:
                from ..allocator import symmetric_mem_pool

                self._pool = symmetric_mem_pool()
            with torch.cuda.use_mem_pool(self._pool):
                return torch.zeros(numel, dtype=dtype, device=self.device)
        return torch.zeros(numel, dtype=dtype, device=self.device)

    def _build_unit(self, u: _Unit, sync_init: bool) -> None:
        off = 0
        for p in u.params:
            u.offsets.append(off)
            off += -(-p.numel() // _ALIGN) * _ALIGN
        quantum = self.world * _ALIGN
        u.numel = max(quantum, -(-off // quantum) * quantum)
        dtype = u.params[0].dtype
        if any(p.dtype != dtype for p in u.params):
            raise ValueError(f"unit {u.name}: parameters of one unit must share a dtype")
        u.full = self._alloc(u.numel, dtype, symmetric=True)
        u.grad = self._alloc(u.numel, dtype, symmetric=True)  # owners reduce straight out of the peers' buffers
        shard = u.numel // self.world
        u.exp_avg = torch.zeros(shard, dtype=dtype, device=self.device)
        u.exp_avg_sq = torch.zeros(shard, dtype=dtype, device=self.device)
        with torch.no_grad():
            for p, o in zip(u.params, u.offsets):
                view = u.full[o : o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                gview = u.grad[o : o + p.numel()].view(p.shape)
                p._mb_grad_view = gview
                if getattr(p, "_mb_linear_weight", False):
                    p._mb_grad_slot = GradSlot(gview)
        if sync_init and self.world > 1:
            dist.broadcast(u.full, src=dist.get_global_rank(self.group, 0), group=self.group)

    # ---- forward side ----------------------------------------------------------------------------
    def _make_pre_hook(self, index: int):
        def hook(module, args, kwargs):
            u = self.units[index]
            if u.ready is not None:
                torch.cuda.current_stream().wait_event(u.ready)
                u.ready = None
            if not torch.is_grad_enabled():
                return None
            u.reduced = False
            new_args = tuple(
                _Boundary.apply(a, self, index) if isinstance(a, torch.Tensor) and a.requires_grad else a for a in args
            )
            return new_args, kwargs

        return hook

    # ---- backward side ---------------------------------------------------------------------------
    def _unit_backward_done(self, index: int) -> None:
        u = self.units[index]
        if u.reduced:
            return
        u.reduced = True
        for p in u.params:
            slot = getattr(p, "_mb_grad_slot", None)
            if slot is not None and slot.written:
                slot.written = False
                if p.grad is not None:  # a second use went through autograd's accumulation
                    p._mb_grad_view.add_(p.grad)
                    p.grad = None
            elif p.grad is not None:
                p._mb_grad_view.copy_(p.grad)
                p.grad = None
            else:
                p._mb_grad_view.zero_()
        self._reduce_and_update(u)

    def _reduce_and_update(self, u: _Unit) -> None:
        step = self.step_count + 1
        shard_n = u.numel // self.world
        pshard = u.full[self.rank * shard_n : (self.rank + 1) * shard_n]
        if not self.cuda:
            self._update_host(u, pshard, step)
            return
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(done)
            if self.world == 1:
                g = u.grad
            elif self._moodist is not None:
                g = torch.empty(shard_n, dtype=torch.float32, device=self.device)
                # bf16 partials cross NVLink, the sum runs in fp32 and the 1/world average is folded in
                self._moodist.reduce_scatter_cast(g, u.grad, int(dist.ReduceOp.AVG), 1.0)
            else:
                g32 = u.grad.float()
                g = torch.empty(shard_n, dtype=torch.float32, device=self.device)
                dist.reduce_scatter_tensor(g, g32, op=dist.ReduceOp.AVG, group=self.group)
            adamw_(pshard, g, u.exp_avg, u.exp_avg_sq, self.lr, self.betas, self.eps, self.weight_decay, step)
            if self.world > 1:
                dist.all_gather_into_tensor(u.full, pshard, group=self.group)
            u.ready = torch.cuda.Event()
            u.ready.record()

    def _update_host(self, u: _Unit, pshard, step) -> None:
        shard_n = u.numel // self.world
        if self.world > 1:
            g = torch.empty(shard_n, dtype=torch.float32)
            g32 = u.grad.float()
            dist.reduce_scatter_tensor(g, g32, op=dist.ReduceOp.SUM, group=self.group)
            g /= self.world
        else:
            g = u.grad
        adamw_(pshard, g, u.exp_avg, u.exp_avg_sq, self.lr, self.betas, self.eps, self.weight_decay, step)
        if self.world > 1:
            gathered = torch.empty_like(u.full)
            dist.all_gather_into_tensor(gathered, pshard.clone(), group=self.group)
            u.full.copy_(gathered)

    def finish_step(self) -> None:
        """Call after ``loss.backward()``: handles the units whose inputs carry no gradient (the embedding)
        and closes the optimizer step."""
        for index in reversed(range(len(self.units))):
            if not self.units[index].reduced:
                self._unit_backward_done(index)
        self.step_count += 1

    def wait(self) -> None:
        """Make the current stream wait for every pending parameter update (before reading parameters
        outside a forward pass, e.g. for evaluation or a checkpoint)."""
        for u in self.units:
            if u.ready is not None:
                torch.cuda.current_stream().wait_event(u.ready)
                u.ready = None

    # ---- checkpointing -----------------------------------------------------------------------------
    def state_dict(self) -> dict:
        """This rank's shard of parameters and optimizer moments per unit, plus the step count."""
        if self.cuda:
            self.wait()
        out = {"step": self.step_count, "world": self.world, "units": {}}
        for u in self.units:
            n = u.numel // self.world
            out["units"][u.name] = {
                "param": u.full[self.rank * n : (self.rank + 1) * n].clone(),
                "exp_avg": u.exp_avg.clone(),
                "exp_avg_sq": u.exp_avg_sq.clone(),
            }
        return out

    def load_state_dict(self, state: dict) -> None:
        if state["world"] != self.world:
            raise ValueError(f"checkpoint was written by {state['world']} ranks, this group has {self.world}")
        self.step_count = int(state["step"])
        for u in self.units:
            s = state["units"][u.name]
            n = u.numel // self.world
            pshard = u.full[self.rank * n : (self.rank + 1) * n]
            with torch.no_grad():
                pshard.copy_(s["param"])
                u.exp_avg.copy_(s["exp_avg"])
                u.exp_avg_sq.copy_(s["exp_avg_sq"])
                if self.world > 1:
                    if self.cuda:
                        dist.all_gather_into_tensor(u.full, pshard, group=self.group)
                    else:
                        gathered = torch.empty_like(u.full)
                        dist.all_gather_into_tensor(gathered, pshard.clone(), group=self.group)
                        u.full.copy_(gathered)
