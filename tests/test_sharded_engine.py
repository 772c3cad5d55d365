"""The sharded engine's host-side logic on CPU ranks over the moodist host backend: after a few steps the
parameters of every rank equal those of a single process that runs AdamW on the rank-averaged gradient,
and a checkpoint written mid-run resumes to the same parameters."""

import copy

import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _tiny_model():
    from moodist_b200.models.llama import Llama, LlamaConfig

    cfg = LlamaConfig(vocab_size=96, dim=32, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=64, max_seq_len=16)
    torch.manual_seed(0)
    model = Llama(cfg, device="cpu").float()
    model.init_weights(0)
    return cfg, model


def _units(m):
    return [("embed", [m.embed])] + [(f"layers.{i}", [l]) for i, l in enumerate(m.layers)] + [("head", [m.norm, m.lm_head])]


def _batch(rank, step, cfg):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randint(0, cfg.vocab_size, (2, 9), generator=g)


def _engine_run(rank, world, port, steps, resume_at):
    from moodist_b200.models.llama import loss_fn
    from moodist_b200.parallel.sharded import ShardedEngine

    dist = init_moodist(rank, world, port)
    cfg, model = _tiny_model()
    ref = copy.deepcopy(model)
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    eng = ShardedEngine(_units(model), **hp)
    opt = torch.optim.AdamW(ref.parameters(), **hp)
    saved = None
    for step in range(steps):
        tok = _batch(rank, step, cfg)
        loss = loss_fn(model(tok[:, :-1]), tok[:, 1:])
        loss.backward()
        eng.finish_step()
        assert all(p.grad is None for p in model.parameters())
        # oracle: every rank's batch in one process, gradients averaged
        opt.zero_grad()
        for r in range(world):
            t = _batch(r, step, cfg)
            (loss_fn(ref(t[:, :-1]), t[:, 1:]) / world).backward()
        opt.step()
        if step + 1 == resume_at:
            saved = copy.deepcopy(eng.state_dict())
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p, q, rtol=2e-4, atol=2e-5, msg=lambda m, n=n: f"{n}: {m}")
    assert eng.step_count == steps
    # resume from the checkpoint with a fresh engine and replay the remaining steps
    cfg2, model2 = _tiny_model()
    eng2 = ShardedEngine(_units(model2), **hp)
    eng2.load_state_dict(saved)
    for step in range(resume_at, steps):
        tok = _batch(rank, step, cfg2)
        loss_fn(model2(tok[:, :-1]), tok[:, 1:]).backward()
        eng2.finish_step()
    for (n, p), (_, q) in zip(model2.named_parameters(), model.named_parameters()):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-7, msg=lambda m, n=n: f"resume {n}: {m}")
    dist.barrier()
    dist.destroy_process_group()


def test_engine_matches_single_process_adamw_world2():
    run_ranks(_engine_run, 2, 4, 2, timeout=180)


def test_engine_world1():
    run_ranks(_engine_run, 1, 3, 1, timeout=180)


def test_engine_world3_uneven_padding():
    run_ranks(_engine_run, 3, 3, 2, timeout=180)


def test_train_ops_cpu_reference_paths():
    """The CPU arithmetic used by those ranks agrees with the textbook formulas."""
    import torch.nn.functional as F

    from moodist_b200.models.llama import apply_rope, rope_tables
    from moodist_b200.ops.train import adamw_, rope_qkv_, swiglu

    torch.manual_seed(0)
    B, S, H, KV, D = 2, 8, 4, 2, 16
    qkv = torch.randn(B, S, (H + 2 * KV) * D)
    cos, sin = rope_tables(D, S, 10000.0, "cpu")
    want_q = apply_rope(qkv[..., : H * D].reshape(B, S, H, D), cos, sin)
    want_k = apply_rope(qkv[..., H * D : (H + KV) * D].reshape(B, S, KV, D), cos, sin)
    v_before = qkv[..., (H + KV) * D :].clone()
    x = qkv.clone().requires_grad_(True)
    out = rope_qkv_(x * 1.0, cos, sin, H + KV, D)
    torch.testing.assert_close(out[..., : H * D].reshape(B, S, H, D), want_q)
    torch.testing.assert_close(out[..., H * D : (H + KV) * D].reshape(B, S, KV, D), want_k)
    assert torch.equal(out[..., (H + KV) * D :], v_before)
    # the rotation is orthogonal: backward of sum(out * w) is the inverse rotation of w
    w = torch.randn_like(qkv)
    (out * w).sum().backward()
    y = qkv.clone().requires_grad_(True)
    q2 = apply_rope(y[..., : H * D].reshape(B, S, H, D), cos, sin).reshape(B, S, H * D)
    k2 = apply_rope(y[..., H * D : (H + KV) * D].reshape(B, S, KV, D), cos, sin).reshape(B, S, KV * D)
    (torch.cat([q2, k2, y[..., (H + KV) * D :]], dim=-1) * w).sum().backward()
    torch.testing.assert_close(x.grad, y.grad)

    gu = torch.randn(5, 24, requires_grad=True)
    g, u = gu.chunk(2, dim=-1)
    ref = F.silu(g) * u
    got = swiglu(gu)
    torch.testing.assert_close(got, ref)
    dy = torch.randn_like(ref)
    (gr,) = torch.autograd.grad(ref, gu, dy, retain_graph=True)
    (gg,) = torch.autograd.grad(got, gu, dy)
    torch.testing.assert_close(gg, gr)

    p = torch.randn(64)
    grad = torch.randn(64)
    q = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(64), torch.zeros(64)
    for step in range(1, 4):
        q.grad = grad.clone()
        opt.step()
        adamw_(p, grad, m, v, 1e-2, (0.9, 0.95), 1e-8, 0.1, step)
    torch.testing.assert_close(p, q.detach(), rtol=1e-5, atol=1e-6)
