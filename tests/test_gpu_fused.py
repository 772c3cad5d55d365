"""Fused collective GEMMs on 2, 4 and 8 GPUs against torch.matmul of the gathered / reduced operands (fp32)."""

import pytest
import torch

from moodist_b200.utils.testing import init_moodist, run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _fused(rank, world, port):
    dist = init_moodist(rank, world, port, device="cuda")
    import moodist_b200 as moodist
    from moodist_b200.ops import fused

    dev = torch.device("cuda", rank)
    pg = moodist.get_backend()

    def shards(rows, cols, seed):
        g = torch.Generator().manual_seed(seed)
        return [(torch.randn(rows, cols, generator=g) * 0.5).bfloat16() for _ in range(world)]

    for it, (m, N, K) in enumerate([(128, 256, 64), (256, 512, 256), (1024, 1536, 1024), (2048, 768, 4096)]):
        # all-gather of activations -> GEMM
        xs = shards(m, K, 10 + it)
        w = shards(N, K, 20 + it)[0].to(dev)
        y, gathered = fused.ag_gemm(pg, xs[rank].to(dev), w)
        ref = torch.cat(xs).float().to(dev) @ w.float().t()
        rel = ((y.float() - ref).abs().max() / ref.abs().max()).item()
        assert rel < 1e-2, ("ag_gemm activations", m, N, K, rel)
        assert torch.equal(gathered.cpu(), torch.cat(xs)), "gathered operand"
        # all-gather of weights -> GEMM (the FSDP shape: weight rows sharded)
        n = 256 * (1 + it % 2)
        ws = shards(n, K, 30 + it)
        x = shards(m, K, 40 + it)[rank].to(dev)
        y, _ = fused.ag_gemm(pg, ws[rank].to(dev), x, gather_weight=True)
        ref = x.float() @ torch.cat(ws).float().to(dev).t()
        rel = ((y.float() - ref).abs().max() / ref.abs().max()).item()
        assert rel < 1e-2, ("ag_gemm weights", m, n, K, rel)
        # GEMM -> reduce-scatter over rows
        M = m * world
        a_all = shards(M, K, 50 + it)
        b_all = shards(N, K, 60 + it)
        out = fused.gemm_rs(pg, a_all[rank].to(dev), b_all[rank].to(dev))
        ref = sum(a_all[r].float() @ b_all[r].float().t() for r in range(world))[rank * m:(rank + 1) * m].to(dev)
        rel = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        assert rel < 2e-2, ("gemm_rs", M, N, K, rel)
    # interleaved with ordinary collectives, repeated (staging halves and counters are reused correctly)
    for i in range(6):
        xs = shards(256, 512, 100 + i)
        w = shards(512, 512, 200 + i)[0].to(dev)
        y, _ = fused.ag_gemm(pg, xs[rank].to(dev), w)
        t = torch.ones(1000, device=dev)
        dist.all_reduce(t)
        a_all, b_all = shards(256 * world, 512, 300 + i), shards(256, 512, 400 + i)
        out = fused.gemm_rs(pg, a_all[rank].to(dev), b_all[rank].to(dev))
        ref = torch.cat(xs).float().to(dev) @ w.float().t()
        assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2
        ref = sum(a_all[r].float() @ b_all[r].float().t() for r in range(world))[rank * 256:(rank + 1) * 256].to(dev)
        assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
        assert bool((t == world).all())
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gemm_collectives(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks(_fused, world, timeout=300, env={"MOODIST_DEVICE_TIMEOUT_MS": 5000})
