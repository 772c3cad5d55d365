"""Fully sharded data parallelism with the re-gather schedule (what torch calls FSDP2 / ``fully_shard``).

Every matrix parameter is sharded by rows at rest: rank ``r`` keeps rows ``[r * rows, (r + 1) * rows)`` of a
weight ``[N, K]`` together with its slice of the optimizer state.  A unit (the embedding, one transformer
block, or the head) gets its full weights only while it computes — once in the forward pass and once
more in the backward pass — and the buffers that held them are reused by the unit after next.  Per unit:

forward
    * weights marked *fused* (the QKV and the gate/up projections of a block) are never gathered by a
      separate collective: ``ops.fused.ag_gemm`` pushes this rank's rows to every peer from inside the GEMM
      kernel and the tile loop consumes the rows as they land, own rows first;
    * the other weights are all-gathered on a side stream one unit ahead, straight out of the peers' shards
      (they live in the symmetric heap) into one of two buffer sets.
backward
    * all matrix weights of the unit are gathered again one unit ahead on the side stream;
    * each weight-gradient GEMM writes a full ``[N, K]`` bf16 gradient, which leaves at once through a
      reduce-scatter that sums in fp32, folds the ``1 / world`` average in and hands this rank an fp32
      gradient of its rows; when the unit's last gradient is in, AdamW updates the unit's shards.

So the only collectives on the critical path are the ones fused into a GEMM; everything else rides on the
side stream under the compute of the neighbouring unit.  One-dimensional parameters (norm weights, a few
thousandths of a percent of the model) are kept whole on every rank in one flat buffer and updated like a
single small resident unit: reduce-scatter, AdamW on the slice, all-gather in place.

With a backend other than this library's (``nccl`` in the benchmark's comparison arm, ``gloo`` or the host
path on CPU ranks in tests) nothing is fused: the same schedule runs with plain collectives.

The reference library ships no trainer; it is benchmarked under torch's FSDP2, whose per-layer
``all_gather_into_tensor`` / ``reduce_scatter_tensor`` calls (reference ``core/processgroup.cc:1059-1284``,
``:1290-1668``) are the collectives this engine issues or fuses.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops.train import adamw_, adamw_master_

_ALIGN = 128  # elements


def _mm(a, b, trans_a=False, trans_b=False, out=None):
    """``op(a) @ op(b).T`` (the contract of ``ops.gemm.gemm``) on the tcgen05 kernel or, on CPU ranks, torch."""
    if a.is_cuda:
        from ..ops.gemm import gemm

        return gemm(a, b, trans_a=trans_a, trans_b=trans_b, out=out)
    aa = a.t() if trans_a else a
    bb = b if trans_b else b.t()
    if out is None:
        return aa @ bb
    torch.matmul(aa, bb, out=out)
    return out


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.stride(0) * t2.element_size()) % 16 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


class _Weight:
    """One row-sharded matrix parameter and where its pieces live."""

    def __init__(self, engine, unit, index, name, module, param, kind):
        self.engine, self.unit, self.index, self.name, self.module, self.kind = engine, unit, index, name, module, kind
        self.param = param
        self.n, self.k = param.shape
        w = engine.world
        self.rows = -(-self.n // w)
        self.n_pad = self.rows * w
        self.fused = False      # forward gather happens inside the GEMM kernel
        self.shard = None       # [rows, k] this rank's rows (symmetric heap on GPUs)
        self.exp_avg = None
        self.exp_avg_sq = None
        self.gshard = None      # fp32 [rows, k] reduced gradient (world > 1)

    # ---- module-facing entry points ----
    def linear(self, x: torch.Tensor) -> torch.Tensor:
        return _LinearFn.apply(x, self, self.engine._dummy)

    def embedding(self, tokens: torch.Tensor) -> torch.Tensor:
        return _EmbeddingFn.apply(tokens, self, self.engine._dummy)


class _LinearFn(torch.autograd.Function):
    """``x @ W.T`` for a weight owned by the engine; the weight gradient leaves through the engine."""

    @staticmethod
    def forward(ctx, x, h, dummy):
        x2 = _rows2d(x)
        y = torch.empty(*x.shape[:-1], h.n, device=x.device, dtype=x.dtype)
        h.engine._linear_forward(h, x2, y.view(-1, h.n))
        ctx.h = h
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, gy):
        h = ctx.h
        (x,) = ctx.saved_tensors
        eng = h.engine
        gy2, x2 = _rows2d(gy), _rows2d(x)
        w = eng._weight_for_backward(h)
        gx = None
        if ctx.needs_input_grad[0]:
            gx = _mm(gy2, w[: h.n], trans_b=True).view(x.shape)  # dx[T, K] = dy[T, N] @ W[N, K]
        gbuf = eng._grad_buffer(h)
        _mm(gy2, x2, trans_a=True, trans_b=True, out=gbuf[: h.n])  # dW[N, K] = dy^T @ x
        eng._grad_ready(h, gbuf)
        return gx, None, None


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, h, dummy):
        w = h.engine._weight_for_forward(h)
        ctx.h = h
        ctx.save_for_backward(tokens)
        return F.embedding(tokens, w)

    @staticmethod
    def backward(ctx, gy):
        h = ctx.h
        (tokens,) = ctx.saved_tensors
        eng = h.engine
        eng._begin_backward(h.unit)
        g2 = gy.reshape(-1, gy.shape[-1])
        # dense [n_pad, K] gradient; torch's kernel sums duplicate tokens in fp32 before rounding
        dense = torch.ops.aten.embedding_dense_backward(g2, tokens.reshape(-1), h.n_pad, -1, False)
        eng._grad_ready(h, dense, pooled=False)
        return None, None, None


class _BufferSet:
    """Gathered weights (and full gradients) of one unit at a time; two sets alternate between neighbours."""

    def __init__(self):
        self.full = {}        # weight index -> [n_pad, k]
        self.owner = {}       # weight index -> (unit index, version) whose weights the buffer holds
        self.gathered = {}    # weight index -> event recorded on the side stream after the gather
        self.grad = {}        # weight index -> [n_pad, k] gradient buffer
        self.grad_free = {}   # weight index -> event: the reduce-scatter that read the buffer is done


class _Unit:
    def __init__(self, index, name):
        self.index, self.name = index, name
        self.weights: list[_Weight] = []
        self.key = None
        self.bufset: _BufferSet | None = None
        self.version = 0          # bumps with every optimizer update of the shards
        self.updated = None       # event on the side stream: shards of the coming step are in place
        self.bwd_begun = False
        self.pending = 0          # gradients still to come in this backward pass
        self.last_fused = None    # the fused weight used last in the forward pass


class RegatherEngine:
    """Shards ``units`` over ``group`` with the re-gather schedule; see the module docstring.

    ``units`` is a list of ``(name, [modules])`` in forward execution order.  Matrix parameters must belong to
    modules that hand their matmul to the engine (``ops.gemm.Linear``, ``models.llama.Embedding``); every other
    parameter is treated as small and kept whole.  ``fused=True`` uses the all-gather GEMM for the weights of
    modules flagged ``_mb_fuse_gather`` whenever the group is this library's and the shape allows it.
    """

    def __init__(self, units, group=None, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True,
                 symmetric_memory=True, sync_init=True, param_names=None, master_weights=False):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        # master_weights: every shard also exists in fp32 with fp32 AdamW moments (what a mixed-precision FSDP2
        # run keeps); the bf16 shard the GEMMs and gathers read is the rounded master. Default off: bf16 shards
        # updated in place with bf16 moments by the single-pass kernel.
        self.master_weights = bool(master_weights)
        self.step_count = 0
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
        self._dummy = torch.zeros((), device=self.device, requires_grad=True)
        self.fused = bool(fused and self._moodist is not None)
        self.fused_calls = 0
        self.exposed_events = None  # list of (before, after) event pairs when profiling the forward/backward waits
        self.units: list[_Unit] = []
        self._small = []  # parameters kept whole
        self._small_master = None
        self._step_open = False
        self._fwd_cursor = -1  # unit whose forward is in progress
        names = param_names or {}
        seen = set()
        for index, (name, mods) in enumerate(units):
            u = _Unit(index, name)
            for m in mods:
                for mod_name, mod in m.named_modules():
                    for pname, p in mod.named_parameters(recurse=False):
                        if id(p) in seen:
                            continue
                        seen.add(id(p))
                        kind = getattr(mod, "_mb_regather_kind", None)
                        if kind is not None and p.dim() == 2 and pname == "weight":
                            full_name = names.get(id(p)) or f"{name}.{mod_name}.{pname}".replace("..", ".")
                            h = _Weight(self, u, len(u.weights), full_name, mod, p, kind)
                            u.weights.append(h)
                        else:
                            self._small.append(p)
            self.units.append(u)
        self._build(sync_init)

    # ---- construction ----------------------------------------------------------------------------
    def _alloc(self, shape, dtype, symmetric=False):
        if symmetric and self._symmetric:
            if self._pool is None:
                from ..allocator import symmetric_mem_pool

                self._pool = symmetric_mem_pool()
            with torch.cuda.use_mem_pool(self._pool):
                return torch.zeros(shape, dtype=dtype, device=self.device)
        return torch.zeros(shape, dtype=dtype, device=self.device)

    def _can_fuse(self, h: _Weight) -> bool:
        if not (self.fused and h.kind == "linear" and getattr(h.module, "_mb_fuse_gather", False)):
            return False
        if h.param.dtype != torch.bfloat16 or h.n != h.n_pad:
            return False
        # the kernel walks 256-row tiles of the gathered operand shard by shard
        return h.n % (self.world * 256) == 0 and h.k % 8 == 0

    def _build(self, sync_init: bool) -> None:
        w, r = self.world, self.rank
        src = dist.get_global_rank(self.group, 0) if w > 1 else 0
        for u in self.units:
            for h in u.weights:
                p = h.param
                if sync_init and w > 1:
                    dist.broadcast(p.data, src=src, group=self.group)
                h.shard = self._alloc((h.rows, h.k), p.dtype, symmetric=True)
                lo, hi = r * h.rows, min(h.n, (r + 1) * h.rows)
                with torch.no_grad():
                    if hi > lo:
                        h.shard[: hi - lo].copy_(p.data[lo:hi])
                state_dtype = torch.float32 if self.master_weights else h.shard.dtype
                h.exp_avg = torch.zeros_like(h.shard, dtype=state_dtype)
                h.exp_avg_sq = torch.zeros_like(h.shard, dtype=state_dtype)
                h.master = h.shard.to(torch.float32, copy=True) if self.master_weights else None
                if w > 1:
                    h.gshard = torch.zeros((h.rows, h.k), dtype=torch.float32, device=self.device)
                p.data = h.shard  # the parameter now *is* this rank's rows
                p.requires_grad_(False)
                p._mb_weight = h
                h.fused = self._can_fuse(h)
                h.module.__dict__["_mb_handle"] = h
            u.key = tuple((h.n_pad, h.k, h.param.dtype, h.kind) for h in u.weights)
        # two buffer sets per distinct unit shape; a shape that occurs once gets one
        by_key: dict = {}
        for u in self.units:
            by_key.setdefault(u.key, []).append(u)
        for key, us in by_key.items():
            sets = [_BufferSet() for _ in range(min(2, len(us)))]
            for i, u in enumerate(us):
                u.bufset = sets[i % len(sets)]
            for s in sets:
                for i, (n_pad, k, dtype, _kind) in enumerate(key):
                    if w > 1:
                        s.full[i] = self._alloc((n_pad, k), dtype)
                    hw = us[0].weights[i]
                    if hw.kind == "linear":
                        # peers read the gradient in place during the reduce-scatter
                        s.grad[i] = self._alloc((n_pad, k), dtype, symmetric=True)
        # small parameters: one flat buffer, whole on every rank
        self._small_numel = 0
        self._small_offsets = []
        for p in self._small:
            self._small_offsets.append(self._small_numel)
            self._small_numel += -(-p.numel() // _ALIGN) * _ALIGN
        if self._small:
            q = w * _ALIGN
            self._small_numel = -(-self._small_numel // q) * q
            dtype = self._small[0].dtype
            self._small_full = self._alloc((self._small_numel,), dtype, symmetric=True)
            self._small_grad = self._alloc((self._small_numel,), dtype, symmetric=True)
            n = self._small_numel // w
            state_dtype = torch.float32 if self.master_weights else dtype
            self._small_m = torch.zeros(n, dtype=state_dtype, device=self.device)
            self._small_v = torch.zeros(n, dtype=state_dtype, device=self.device)
            with torch.no_grad():
                for p, o in zip(self._small, self._small_offsets):
                    view = self._small_full[o : o + p.numel()].view(p.shape)
                    view.copy_(p.data)
                    p.data = view
            if sync_init and w > 1:
                dist.broadcast(self._small_full, src=src, group=self.group)
            n = self._small_numel // w
            if self.master_weights:
                self._small_master = self._small_full[r * n : (r + 1) * n].to(torch.float32, copy=True)
        self._small_ready = None

    # ---- stream helpers ----------------------------------------------------------------------------
    def _side(self):
        """Context in which collectives and optimizer kernels are issued: the side stream, after everything
        the compute stream has been given so far."""
        if not self.cuda:
            import contextlib

            return contextlib.nullcontext()
        ev = torch.cuda.Event()
        ev.record()
        self.comm_stream.wait_event(ev)
        return torch.cuda.stream(self.comm_stream)

    def _wait_on_compute(self, ev) -> None:
        if ev is None or not self.cuda:
            return
        cur = torch.cuda.current_stream()
        if self.exposed_events is not None:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            cur.wait_event(ev)
            b.record()
            self.exposed_events.append((a, b))
        else:
            cur.wait_event(ev)

    def _all_gather(self, out, shard) -> None:
        if self._moodist is not None:
            self._moodist.all_gather_cast(out, shard)
        else:
            dist.all_gather_into_tensor(out, shard, group=self.group)

    # ---- gathers ----------------------------------------------------------------------------------
    def _issue_gathers(self, index: int, forward: bool) -> None:
        """Queue, on the side stream, the all-gathers unit ``index`` needs for the pass that is coming."""
        if self.world == 1 or index < 0 or index >= len(self.units):
            return
        u = self.units[index]
        todo = []
        for h in u.weights:
            if forward and h.fused:
                continue
            if not forward and h.kind == "embedding":
                continue  # its backward needs the token ids only
            if u.bufset.owner.get(h.index) == (u.index, u.version):
                continue
            todo.append(h)
        if not todo:
            return
        with self._side():
            for h in todo:
                self._all_gather(u.bufset.full[h.index], h.shard)
                u.bufset.owner[h.index] = (u.index, u.version)
                if self.cuda:
                    ev = torch.cuda.Event()
                    ev.record()
                    u.bufset.gathered[h.index] = ev

    def _begin_step(self) -> None:
        if self._step_open:
            return
        self._step_open = True
        for u in self.units:
            u.bwd_begun = False
        if self._small_ready is not None:
            self._wait_on_compute(self._small_ready)
            self._small_ready = None

    def _begin_forward(self, u: _Unit) -> None:
        if self._fwd_cursor == u.index:
            return
        self._begin_step()
        self._fwd_cursor = u.index
        u.last_fused = None
        if u.updated is not None:
            # the fused kernel reads this rank's shard on the compute stream
            self._wait_on_compute(u.updated)
            u.updated = None
        self._issue_gathers(u.index, True)
        fused = [h for h in u.weights if h.fused]
        if fused:
            u.last_fused = fused[-1]  # weights are listed in module order, which is the order of use
        else:
            self._issue_gathers(u.index + 1, True)

    def _weight_for_forward(self, h: _Weight) -> torch.Tensor:
        u = h.unit
        self._begin_forward(u)
        if self.world == 1:
            return h.shard
        assert u.bufset.owner.get(h.index) == (u.index, u.version), f"{h.name}: gathered weight missing"
        self._wait_on_compute(u.bufset.gathered.pop(h.index, None))
        return u.bufset.full[h.index]

    def _linear_forward(self, h: _Weight, x2, y2) -> None:
        u = h.unit
        self._begin_forward(u)
        if h.fused and self.world > 1:
            from ..ops.fused import ag_gemm

            ag_gemm(self._moodist, h.shard, x2, gather_weight=True, out=y2)
            self.fused_calls += 1
            if u.last_fused is h:
                # the next unit's plain gathers queue up behind this kernel and run under what follows it
                self._issue_gathers(u.index + 1, True)
            return
        w = self._weight_for_forward(h)
        _mm(x2, w[: h.n], out=y2)

    # ---- backward ---------------------------------------------------------------------------------
    def _begin_backward(self, u: _Unit) -> None:
        if u.bwd_begun:
            if u.pending == 0:
                # every gradient of the unit has been reduced and applied already: this is a second backward
                # pass (or a weight used twice) within one optimizer step, which this schedule cannot serve
                raise RuntimeError(f"unit {u.name}: a second backward pass before finish_step(); the re-gather engine "
                                   "applies each weight's gradient as soon as it is produced (one backward per step, "
                                   "every weight used once)")
            return
        u.bwd_begun = True
        self._fwd_cursor = -1
        u.pending = len(u.weights)
        self._issue_gathers(u.index, False)
        self._issue_gathers(u.index - 1, False)

    def _weight_for_backward(self, h: _Weight) -> torch.Tensor:
        u = h.unit
        self._begin_backward(u)
        if self.world == 1:
            return h.shard
        assert u.bufset.owner.get(h.index) == (u.index, u.version), f"{h.name}: gathered weight missing"
        self._wait_on_compute(u.bufset.gathered.pop(h.index, None))
        return u.bufset.full[h.index]

    def _grad_buffer(self, h: _Weight) -> torch.Tensor:
        s = h.unit.bufset
        self._wait_on_compute(s.grad_free.pop(h.index, None))
        return s.grad[h.index]

    def _grad_ready(self, h: _Weight, g: torch.Tensor, pooled: bool = True) -> None:
        """``g`` is the full ``[n_pad, k]`` gradient of ``h`` (rows past ``n`` are zero): reduce it, and when it is
        the unit's last, update the unit's shards."""
        u = h.unit
        with self._side():
            if self.world > 1:
                self._reduce_scatter(h.gshard, g)
                grad = h.gshard
            else:
                grad = g
            step = self.step_count + 1
            self._adamw(h.shard.view(-1), h.master, grad.reshape(-1), h.exp_avg.view(-1), h.exp_avg_sq.view(-1), step)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record()
                if pooled:
                    u.bufset.grad_free[h.index] = ev
                else:
                    g.record_stream(self.comm_stream)
        u.pending -= 1
        if u.pending == 0:
            u.version += 1
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                u.updated = ev

    def _adamw(self, p, master, g, m, v, step) -> None:
        if master is not None:
            adamw_master_(p, master.view(-1), g, m, v, self.lr, self.betas, self.eps, self.weight_decay, step)
        else:
            adamw_(p, g, m, v, self.lr, self.betas, self.eps, self.weight_decay, step)

    def _reduce_scatter(self, out32, g) -> None:
        if self._moodist is not None:
            # bf16 partial gradients cross NVLink, the sum runs in fp32 and the 1/world average is folded in
            self._moodist.reduce_scatter_cast(out32.view(-1), g.view(-1), int(dist.ReduceOp.AVG), 1.0)
        elif self.cuda:
            dist.reduce_scatter_tensor(out32.view(-1), g.float().view(-1), op=dist.ReduceOp.AVG, group=self.group)
        else:
            dist.reduce_scatter_tensor(out32.view(-1), g.float().view(-1), op=dist.ReduceOp.SUM, group=self.group)
            out32.div_(self.world)

    # ---- end of step --------------------------------------------------------------------------------
    def finish_step(self) -> None:
        """Call after ``loss.backward()``: updates the small parameters and closes the optimizer step."""
        for u in self.units:
            if u.bwd_begun and u.pending:
                raise RuntimeError(f"unit {u.name}: {u.pending} weight gradients never arrived")
        if self._small:
            self._update_small()
        self.step_count += 1
        self._step_open = False
        self._fwd_cursor = -1
        # the first unit's weights for the coming step are requested now, behind its optimizer update
        if self.units and any(u.bwd_begun for u in self.units):
            self._issue_gathers(0, True)

    def _update_small(self) -> None:
        w = self.world
        n = self._small_numel // w
        with torch.no_grad():
            for p, o in zip(self._small, self._small_offsets):
                gv = self._small_grad[o : o + p.numel()].view(p.shape)
                if p.grad is not None:
                    gv.copy_(p.grad)
                    p.grad = None
                else:
                    gv.zero_()
        pshard = self._small_full[self.rank * n : (self.rank + 1) * n]
        step = self.step_count + 1
        with self._side():
            if w == 1:
                g = self._small_grad
            else:
                g = torch.empty(n, dtype=torch.float32, device=self.device)
                self._reduce_scatter(g, self._small_grad)
            self._adamw(pshard, self._small_master, g, self._small_m, self._small_v, step)
            if w > 1:
                if self.cuda:
                    dist.all_gather_into_tensor(self._small_full, pshard, group=self.group)
                else:
                    gathered = torch.empty_like(self._small_full)
                    dist.all_gather_into_tensor(gathered, pshard.clone(), group=self.group)
                    self._small_full.copy_(gathered)
            if self.cuda:
                self._small_ready = torch.cuda.Event()
                self._small_ready.record()

    def wait(self) -> None:
        """Make the current stream wait for every pending update and gather of the side stream."""
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    def exposed_ms(self) -> float:
        """Sum of the time the compute stream spent waiting for the side stream since profiling was switched
        on (``engine.exposed_events = []``); synchronises the device."""
        torch.cuda.synchronize(self.device)
        total = sum(a.elapsed_time(b) for a, b in (self.exposed_events or []))
        self.exposed_events = [] if self.exposed_events is not None else None
        return float(total)

    # ---- whole parameters, checkpoints ----------------------------------------------------------------
    def full_parameters(self) -> dict:
        """Every parameter whole, by name (a collective: all ranks must call it)."""
        self.wait()
        out = {}
        for u in self.units:
            for h in u.weights:
                if self.world == 1:
                    full = h.shard
                else:
                    full = torch.empty((h.n_pad, h.k), dtype=h.shard.dtype, device=self.device)
                    if self.cuda:
                        dist.all_gather_into_tensor(full, h.shard, group=self.group)
                    else:
                        dist.all_gather_into_tensor(full, h.shard.clone(), group=self.group)
                out[h.name] = full[: h.n].clone()
        return out

    def state_dict(self) -> dict:
        """This rank's rows of every weight with their optimizer moments, the small parameters' slice, and
        the step count."""
        self.wait()
        st = {"step": self.step_count, "world": self.world, "weights": {}, "small": None}
        for u in self.units:
            for h in u.weights:
                st["weights"][h.name] = {"param": h.shard.clone(), "exp_avg": h.exp_avg.clone(),
                                         "exp_avg_sq": h.exp_avg_sq.clone()}
                if h.master is not None:
                    st["weights"][h.name]["master"] = h.master.clone()
        if self._small:
            n = self._small_numel // self.world
            st["small"] = {"param": self._small_full[self.rank * n : (self.rank + 1) * n].clone(),
                           "exp_avg": self._small_m.clone(), "exp_avg_sq": self._small_v.clone()}
            if self._small_master is not None:
                st["small"]["master"] = self._small_master.clone()
        return st

    def load_state_dict(self, state: dict) -> None:
        if state["world"] != self.world:
            raise ValueError(f"checkpoint was written by {state['world']} ranks, this group has {self.world}")
        self.wait()
        self.step_count = int(state["step"])
        with torch.no_grad():
            for u in self.units:
                for h in u.weights:
                    s = state["weights"][h.name]
                    h.shard.copy_(s["param"])
                    h.exp_avg.copy_(s["exp_avg"])
                    h.exp_avg_sq.copy_(s["exp_avg_sq"])
                    if h.master is not None:
                        h.master.copy_(s["master"] if "master" in s else s["param"])
                u.version += 1
            if self._small:
                s = state["small"]
                n = self._small_numel // self.world
                pshard = self._small_full[self.rank * n : (self.rank + 1) * n]
                pshard.copy_(s["param"])
                self._small_m.copy_(s["exp_avg"])
                self._small_v.copy_(s["exp_avg_sq"])
                if self._small_master is not None:
                    self._small_master.copy_(s["master"] if "master" in s else s["param"])
                if self.world > 1:
                    if self.cuda:
                        dist.all_gather_into_tensor(self._small_full, pshard, group=self.group)
                    else:
                        gathered = torch.empty_like(self._small_full)
                        dist.all_gather_into_tensor(gathered, pshard.clone(), group=self.group)
                        self._small_full.copy_(gathered)
