"""tcgen05 GEMM numerics against a plain PyTorch fp32 reference of the same product."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


@pytest.fixture(params=[1, 0], ids=["one_sm", "by_shape"])
def variant(request):
    """Every GEMM test runs on the one-SM kernel and on the shape-based choice (two-SM pairs from 256 rows)."""
    from moodist_b200._core import _C

    old = _C.get_gemm_variant()
    _C.gemm_variant(request.param)
    yield request.param
    _C.gemm_variant(old)


@pytest.mark.parametrize(
    "M,N,K", [(128, 256, 64), (200, 264, 136), (256, 256, 64), (392, 520, 200), (1024, 2048, 1024), (4096, 1536, 4096)]
)
@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_matches_fp32(M, N, K, trans_a, trans_b, variant):
    from moodist_b200.ops.gemm import gemm

    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ain = a.t().contiguous() if trans_a else a
    bin_ = b.t().contiguous() if trans_b else b
    c = gemm(ain, bin_, trans_a=trans_a, trans_b=trans_b)
    ref = _ref(a, b)
    rel = (c.float() - ref).abs().max() / ref.abs().max()
    assert rel < 1e-2, rel
    c32 = gemm(ain, bin_, trans_a=trans_a, trans_b=trans_b, out_fp32=True)
    rel32 = (c32 - ref).abs().max() / ref.abs().max()
    assert rel32 < 1e-5, rel32


def test_gemm_silu_epilogue(variant):
    from moodist_b200.ops.gemm import gemm

    a = torch.randn(512, 512, device="cuda").bfloat16()
    b = torch.randn(512, 512, device="cuda").bfloat16()
    c = gemm(a, b, epilogue=1)
    ref = torch.nn.functional.silu(_ref(a, b))
    assert (c.float() - ref).abs().max() / ref.abs().max() < 1e-2


def test_linear_autograd_matches_torch(variant):
    from moodist_b200.ops.gemm import linear

    torch.manual_seed(0)
    x = torch.randn(4, 96, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad)):
        assert (got.float() - ref).abs().max() / ref.abs().max() < 2e-2


def test_smoke_entry():
    import __graft_entry__ as entry

    entry.smoke()
