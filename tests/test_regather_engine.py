"""The re-gather (FSDP2-style) engine's host-side logic on CPU ranks over the moodist host backend: weights
sharded by rows at rest, gathered per unit for forward and backward, gradients reduce-scattered per weight.
After a few steps every parameter equals that of a single process running AdamW on the rank-averaged
gradient, and a checkpoint written mid-run resumes to the same parameters."""

import copy

import torch

from moodist_b200.utils.testing import init_moodist, run_ranks


def _tiny_model():
    from moodist_b200.models.llama import Llama, LlamaConfig

    cfg = LlamaConfig(vocab_size=96, dim=32, n_layers=3, n_heads=4, n_kv_heads=2, ffn_dim=64, max_seq_len=16)
    torch.manual_seed(0)
    model = Llama(cfg, device="cpu").float()
    model.init_weights(0)
    return cfg, model


def _units(m):
    return [("embed", [m.embed])] + [(f"layers.{i}", [l]) for i, l in enumerate(m.layers)] + [("head", [m.norm, m.lm_head])]


def _batch(rank, step, cfg):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randint(0, cfg.vocab_size, (2, 9), generator=g)


def _engine(model, hp, **kw):
    from moodist_b200.parallel.regather import RegatherEngine

    names = {id(p): n for n, p in model.named_parameters()}
    return RegatherEngine(_units(model), param_names=names, **hp, **kw)


def _check(eng, model, ref, rtol, atol, what=""):
    full = eng.full_parameters()
    for n, q in ref.named_parameters():
        got = full[n] if n in full else dict(model.named_parameters())[n]
        torch.testing.assert_close(got, q, rtol=rtol, atol=atol, msg=lambda m, n=n: f"{what}{n}: {m}")


def _engine_run(rank, world, port, steps, resume_at, master=False):
    from moodist_b200.models.llama import loss_fn

    dist = init_moodist(rank, world, port)
    cfg, model = _tiny_model()
    ref = copy.deepcopy(model)
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    eng = _engine(model, hp, master_weights=master)
    # at rest every matrix parameter is this rank's rows only
    for u in eng.units:
        for h in u.weights:
            assert h.param.shape == (h.rows, h.k) and h.rows * world >= h.n
    opt = torch.optim.AdamW(ref.parameters(), **hp)
    saved = None
    for step in range(steps):
        tok = _batch(rank, step, cfg)
        loss = loss_fn(model(tok[:, :-1]), tok[:, 1:])
        loss.backward()
        eng.finish_step()
        opt.zero_grad()
        ref_loss = None
        for r in range(world):
            t = _batch(r, step, cfg)
            l = loss_fn(ref(t[:, :-1]), t[:, 1:])
            (l / world).backward()
            if r == rank:
                ref_loss = l.item()
        opt.step()
        assert abs(loss.item() - ref_loss) < 1e-4, (step, loss.item(), ref_loss)
        if step + 1 == resume_at:
            saved = copy.deepcopy(eng.state_dict())
    _check(eng, model, ref, 2e-4, 2e-5)
    assert eng.step_count == steps
    # a forward pass without a backward (evaluation) works between steps and twice in a row
    with torch.no_grad():
        tok = _batch(rank, 99, cfg)
        a = model(tok[:, :-1])
        b = model(tok[:, :-1])
        torch.testing.assert_close(a, b)
        torch.testing.assert_close(a, ref(tok[:, :-1]), rtol=1e-3, atol=1e-4)
    # a second backward pass within one step is refused (gradients are applied as they are produced)
    tok = _batch(rank, 98, cfg)
    loss_fn(model(tok[:, :-1]), tok[:, 1:]).backward()
    try:
        loss_fn(model(tok[:, :-1]), tok[:, 1:]).backward()
        raise AssertionError("second backward was accepted")
    except RuntimeError as e:
        assert "second backward" in str(e)
    # resume from the checkpoint with a fresh engine and replay the remaining steps
    cfg2, model2 = _tiny_model()
    eng2 = _engine(model2, hp, master_weights=master)
    eng2.load_state_dict(saved)
    for step in range(resume_at, steps):
        tok = _batch(rank, step, cfg2)
        loss_fn(model2(tok[:, :-1]), tok[:, 1:]).backward()
        eng2.finish_step()
    _check(eng2, model2, ref, 2e-4, 2e-5, "resume ")
    dist.barrier()
    dist.destroy_process_group()


def test_regather_matches_single_process_adamw_world2():
    run_ranks(_engine_run, 2, 4, 2, timeout=180)


def test_regather_world1():
    run_ranks(_engine_run, 1, 3, 1, timeout=180)


def test_regather_world3_padded_rows():
    run_ranks(_engine_run, 3, 3, 2, timeout=180)


def test_regather_with_fp32_master_weights_world2():
    """fp32 master shards and fp32 moments (the torch-op AdamW path): same trajectory as the oracle, and the
    master copies travel through the checkpoint."""
    run_ranks(_engine_run, 2, 4, 2, True, timeout=180)


def test_adamw_master_matches_torch_adamw_and_rounds_into_bf16():
    from moodist_b200.ops.train import adamw_master_

    torch.manual_seed(0)
    master = torch.randn(1000)
    p = master.to(torch.bfloat16)
    q = master.clone().requires_grad_(True)
    opt = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(1000), torch.zeros(1000)
    for step in range(1, 5):
        g = torch.randn(1000)
        q.grad = g.clone()
        opt.step()
        adamw_master_(p, master, g.to(torch.bfloat16) if step % 2 else g, m, v, 1e-2, (0.9, 0.95), 1e-8, 0.1, step)
    torch.testing.assert_close(master, q.detach(), rtol=2e-2, atol=2e-2)  # two of the gradients were rounded to bf16
    assert torch.equal(p, master.to(torch.bfloat16))
