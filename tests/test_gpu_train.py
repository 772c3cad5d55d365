"""Training kernels (rotary embedding, SwiGLU, cross-entropy, AdamW) against fp32 PyTorch references of the
same ops, and the sharded engine on GPUs against a single-process AdamW on rank-averaged gradients."""


import pytest
import torch
import torch.nn.functional as F

from moodist_b200.utils.testing import init_moodist, run_ranks

pytestmark = pytest.mark.gpu


def test_rope_kernel_forward_backward():
    from moodist_b200.models.llama import apply_rope, rope_tables
    from moodist_b200.ops.train import rope_qkv_

    torch.manual_seed(0)
    dev = "cuda"
    B, S, H, KV, D = 2, 96, 8, 2, 128
    cos, sin = rope_tables(D, S, 500000.0, dev)
    base = torch.randn(B, S, (H + 2 * KV) * D, device=dev).bfloat16()
    x = base.clone().requires_grad_(True)
    out = rope_qkv_(x * 1, cos, sin, H + KV, D)
    ref_q = apply_rope(base[..., : H * D].float().view(B, S, H, D), cos, sin).view(B, S, H * D)
    ref_k = apply_rope(base[..., H * D : (H + KV) * D].float().view(B, S, KV, D), cos, sin).view(B, S, KV * D)
    torch.testing.assert_close(out[..., : H * D].float(), ref_q, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(out[..., H * D : (H + KV) * D].float(), ref_k, rtol=1e-2, atol=2e-2)
    assert torch.equal(out[..., (H + KV) * D :], base[..., (H + KV) * D :])
    w = torch.randn_like(base)
    (out.float() * w.float()).sum().backward()
    y = base.float().requires_grad_(True)
    q2 = apply_rope(y[..., : H * D].view(B, S, H, D), cos, sin).reshape(B, S, H * D)
    k2 = apply_rope(y[..., H * D : (H + KV) * D].view(B, S, KV, D), cos, sin).reshape(B, S, KV * D)
    (torch.cat([q2, k2, y[..., (H + KV) * D :]], dim=-1) * w.float()).sum().backward()
    torch.testing.assert_close(x.grad.float(), y.grad, rtol=1e-2, atol=2e-2)


def test_swiglu_kernel_forward_backward():
    from moodist_b200.ops.train import swiglu

    torch.manual_seed(1)
    gu = (torch.randn(3, 130, 2 * 448, device="cuda") * 2).bfloat16().requires_grad_(True)
    out = swiglu(gu)
    g32 = gu.detach().float().requires_grad_(True)
    a, b = g32.chunk(2, dim=-1)
    ref = F.silu(a) * b
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2)
    dy = torch.randn_like(out)
    out.backward(dy)
    ref.backward(dy.float())
    torch.testing.assert_close(gu.grad.float(), g32.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("rows,D", [(5, 256), (777, 4096), (300, 8192), (64, 1000)])
def test_rmsnorm_kernel_forward_backward(rows, D):
    from moodist_b200.ops.train import rms_norm

    torch.manual_seed(rows + D)
    x = (torch.randn(3, rows, D, device="cuda") * 2).bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_(True)
    y = rms_norm(x, w, 1e-5)
    x32 = x.detach().float().requires_grad_(True)
    w32 = w.detach().float().requires_grad_(True)
    ref = F.rms_norm(x32, (D,), w32, 1e-5)
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=1e-2)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float())
    torch.testing.assert_close(x.grad.float(), x32.grad, rtol=2e-2, atol=2e-2)
    # dw sums 3 * rows products: compare relative to its magnitude
    rel = (w.grad.float() - w32.grad).abs().max() / w32.grad.abs().max()
    assert rel < 2e-2, rel


@pytest.mark.parametrize("rows,V", [(37, 1000), (513, 128256), (16, 1003)])
def test_cross_entropy_kernel(rows, V):
    from moodist_b200._core import _C
    from moodist_b200.ops.train import cross_entropy

    torch.manual_seed(2)
    Vpad = -(-V // 8) * 8
    buf = (torch.randn(rows, Vpad, device="cuda") * 3).bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    ref_in = buf[:, :V].float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, tgt)
    ref.backward()
    if V == Vpad:
        logits = buf.clone().requires_grad_(True)
        x = logits * 1
        loss = cross_entropy(x, tgt)
        torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-4)
        (loss * 2.0).backward()
        torch.testing.assert_close(logits.grad.float(), 2.0 * ref_in.grad, rtol=2e-2, atol=1e-6)
    else:
        # a row pitch wider than V: the tail loop handles the last V % 8 columns
        view = buf[:, :V]
        rows_loss, lse = _C.cross_entropy_fwd(view, tgt, -100)
        torch.testing.assert_close(rows_loss.mean(), ref, rtol=1e-4, atol=1e-4)
        _C.cross_entropy_bwd_(view, tgt, lse, torch.ones(1, device="cuda"), 1.0 / rows, -100)
        torch.testing.assert_close(view.float(), ref_in.grad, rtol=2e-2, atol=1e-6)


def test_cross_entropy_ignore_index():
    from moodist_b200.ops.train import cross_entropy

    torch.manual_seed(3)
    logits = torch.randn(64, 512, device="cuda").bfloat16()
    tgt = torch.randint(0, 512, (64,), device="cuda")
    tgt[::3] = -100
    ref = F.cross_entropy(logits.float(), tgt, ignore_index=-100)
    got = cross_entropy(logits.clone(), tgt, ignore_index=-100)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_adamw_kernel(gdtype):
    from moodist_b200.ops.train import adamw_

    torch.manual_seed(4)
    n = 8 * 1000 + 8 * 37
    p0 = torch.randn(n, device="cuda").bfloat16()
    p = p0.clone()
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    q = p0.float().clone().requires_grad_(True)
    opt = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").to(gdtype)
        q.grad = g.float()
        opt.step()
        adamw_(p, g, m, v, 1e-2, (0.9, 0.95), 1e-8, 0.1, step)
    # three updates of size ~lr each, bf16 storage: within a few bf16 ulps of the fp32 trajectory
    torch.testing.assert_close(p.float(), q.detach(), rtol=2e-2, atol=2e-2)
    assert (p.float() - p0.float()).abs().mean() > 5e-3


def _tiny_cfg():
    from moodist_b200.models.llama import LlamaConfig

    return LlamaConfig(vocab_size=1024, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512, max_seq_len=128)


def _trainer_run(rank, world, port, steps, schedule="resident", fused=True):
    from moodist_b200.models.llama import Llama, loss_fn
    from moodist_b200.parallel.fsdp import ShardedTrainer

    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    cfg = _tiny_cfg()
    tr = ShardedTrainer(cfg, lr=1e-3, seed=0, schedule=schedule, fused=fused)
    # oracle on this GPU: same bf16 model, every rank's batch, fp32 AdamW on the averaged gradient is too
    # strict for bf16 weights, so compare losses and parameters with bf16-sized tolerances
    torch.manual_seed(0)
    ref = Llama(cfg, device=dev)
    ref.init_weights(0)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)

    def batch(r, step):
        g = torch.Generator().manual_seed(100 * step + r)
        return torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(dev)

    for step in range(steps):
        loss = tr.step_on_device(batch(rank, step))
        opt.zero_grad()
        ref_losses = []
        for r in range(world):
            t = batch(r, step)
            l = loss_fn(ref(t[:, :-1]), t[:, 1:])
            (l / world).backward()
            ref_losses.append(l.item())
        opt.step()
        assert abs(loss.item() - ref_losses[rank]) < 0.05, (step, loss.item(), ref_losses)
    tr.engine.wait()
    torch.cuda.synchronize()
    worst = 0.0
    if schedule == "regather":
        # at rest a rank holds its rows only: gather every weight for the comparison
        full = tr.engine.full_parameters()
        mine = dict(tr.model.named_parameters())
        for n, q in ref.named_parameters():
            p = full[n] if n in full else mine[n]
            assert p.shape == q.shape, (n, p.shape, q.shape)
            worst = max(worst, (p.float() - q.float()).abs().max().item())
        assert worst < 2e-2, worst
        if world > 1:
            assert all(h.param.shape[0] * world >= h.n and h.param.shape[0] < h.n for u in tr.engine.units for h in u.weights)
            # every weight whose shape allows it (QKV and gate/up of every block) is gathered inside its GEMM
            per_step = sum(h.fused for u in tr.engine.units for h in u.weights)
            assert (per_step > 0) == bool(fused), per_step
            assert tr.engine.fused_calls == per_step * steps, (tr.engine.fused_calls, per_step, steps)
        flat = torch.cat([v.float().reshape(-1) for v in full.values()] + [tr.engine._small_full.float()])
    else:
        for (n, p), (_, q) in zip(tr.model.named_parameters(), ref.named_parameters()):
            worst = max(worst, (p.float() - q.float()).abs().max().item())
        assert worst < 2e-2, worst
        # every rank holds the same gathered parameters
        flat = torch.cat([u.full.float() for u in tr.engine.units])
    lo, hi = flat.clone(), flat.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert torch.equal(lo, hi)
    dist.barrier()
    dist.destroy_process_group()


def test_native_engine_one_gpu():
    run_ranks(_trainer_run, 1, 4, timeout=300)


@pytest.mark.multigpu
def test_native_engine_two_gpus():
    run_ranks(_trainer_run, 2, 4, timeout=300)


def test_regather_engine_one_gpu():
    run_ranks(_trainer_run, 1, 4, "regather", timeout=300)


@pytest.mark.multigpu
@pytest.mark.parametrize("fused", [True, False])
def test_regather_engine_two_gpus(fused):
    """The FSDP2-style schedule on two GPUs (weights gathered inside the QKV / gate-up GEMMs when fused)
    against single-process AdamW on the rank-averaged gradient."""
    run_ranks(_trainer_run, 2, 4, "regather", fused, timeout=300, env={"MOODIST_DEVICE_TIMEOUT_MS": 10000})


@pytest.mark.multigpu
def test_regather_engine_four_gpus():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    run_ranks(_trainer_run, 4, 3, "regather", True, timeout=300, env={"MOODIST_DEVICE_TIMEOUT_MS": 10000})


def _fsdp2_run(rank, world, port):
    from moodist_b200.parallel.fsdp import ShardedTrainer

    dist = init_moodist(rank, world, port, device="cuda")
    dev = torch.device("cuda", rank)
    cfg = _tiny_cfg()
    tr = ShardedTrainer(cfg, lr=1e-3, seed=0, engine="fsdp2")
    g = torch.Generator().manual_seed(rank)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(dev)
    losses = [tr.step_on_device(tok).item() for _ in range(6)]
    assert losses[-1] < losses[0] - 0.05, losses
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_fsdp2_engine_two_gpus():
    run_ranks(_fsdp2_run, 2, timeout=300)
