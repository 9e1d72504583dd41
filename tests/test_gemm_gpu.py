"""GPU: the tcgen05 bf16 GEMM against fp32 matmul of the same bf16 operands."""

import pytest
import torch

from torchtitan_b200.ops import ext

pytestmark = pytest.mark.gpu

SHAPES = [(128, 256, 64), (256, 512, 256), (200, 264, 136), (1024, 768, 4096), (8, 8, 8), (4096, 6144, 512),
          (304, 1000, 72), (2560, 2304, 1088)]


def _operands(mode, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K + mode)
    a = torch.randn((K, M) if mode == 2 else (M, K), device="cuda", generator=g).bfloat16()
    b = torch.randn((N, K) if mode == 0 else (K, N), device="cuda", generator=g).bfloat16()
    af = a.float().t() if mode == 2 else a.float()
    bf = b.float().t() if mode == 0 else b.float()
    return a, b, af @ bf


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_matches_fp32(mode, M, N, K, variant):
    """variant 1 = one CTA per 128x256 tile, variant 2 = CTA pair per 256x256 tile."""
    assert ext.load()
    a, b, ref = _operands(mode, M, N, K)
    c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    torch.ops.tb200.gemm_set_variant(variant)
    try:
        torch.ops.tb200.gemm_bf16(a, b, c, mode, False)
        torch.cuda.synchronize()
    finally:
        torch.ops.tb200.gemm_set_variant(0)
    assert torch.ops.tb200.gemm_status(True) == 0
    err = (c.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-2
    assert err <= tol, (err, tol)


@pytest.mark.parametrize("mode", [0, 2])
def test_gemm_accumulate(mode):
    M, N, K = 384, 520, 192
    a, b, ref = _operands(mode, M, N, K)
    c0 = torch.randn(M, N, device="cuda").bfloat16()
    c = c0.clone()
    torch.ops.tb200.gemm_bf16(a, b, c, mode, True)
    torch.cuda.synchronize()
    exp = c0.float() + ref
    assert (c.float() - exp).abs().max().item() <= 2e-2 * exp.abs().max().item() + 1e-2


def test_linear_layer_through_tcgen05_path():
    from torchtitan_b200.ops import functional as OF

    OF.settings.gemm = "tcgen05"
    try:
        x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_()
        w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
        y = OF.linear(x, w)
        g = torch.randn_like(y)
        y.backward(g)
        xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
        yr = xr @ wr.t()
        yr.backward(g.float())
        assert torch.allclose(y.float(), yr, atol=5e-2, rtol=2e-2)
        assert torch.allclose(x.grad.float(), xr.grad, atol=5e-2, rtol=2e-2)
        assert torch.allclose(w.grad.float(), wr.grad, atol=0.5, rtol=2e-2)
    finally:
        OF.settings.gemm = "cublas"
