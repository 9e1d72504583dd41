"""GPU: grouped tcgen05 GEMM (rows sorted by group, groups padded to the row tile) vs fp32 loops."""

import pytest
import torch

from torchtitan_b200.ops import ext

pytestmark = pytest.mark.gpu


def _layout(counts, align, extra_rows=0):
    padded = [(c + align - 1) // align * align for c in counts]
    offs = [0]
    for p in padded:
        offs.append(offs[-1] + p)
    R = offs[-1] + extra_rows
    valid = torch.zeros(R, dtype=torch.bool)
    for g, c in enumerate(counts):
        valid[offs[g]:offs[g] + c] = True
    return torch.tensor(offs, dtype=torch.int32, device="cuda"), offs, R, valid.cuda()


@pytest.mark.parametrize("align", [128, 256])
@pytest.mark.parametrize("counts,N,K", [([130, 0, 257, 5], 768, 512), ([1000, 300, 0, 0, 64, 700], 256, 2048)])
def test_grouped_forward_and_dgrad(counts, N, K, align):
    ops = ext.require()
    G = len(counts)
    offs_t, offs, R, valid = _layout(counts, align, extra_rows=align)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(R, K, device="cuda", generator=g).bfloat16() * valid[:, None]
    w = (torch.randn(G, N, K, device="cuda", generator=g) * 0.05).bfloat16()
    y = torch.full((R, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped_bf16(x, w, y, offs_t, 0, align, False)
    dy = torch.randn(R, N, device="cuda", generator=g).bfloat16() * valid[:, None]
    dx = torch.full((R, K), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped_bf16(dy, w, dx, offs_t, 1, align, False)
    torch.cuda.synchronize()
    assert ops.gemm_status(True) == 0
    for e in range(G):
        a, b = offs[e], offs[e + 1]
        if a == b:
            continue
        ref = x[a:b].float() @ w[e].float().t()
        assert (y[a:b].float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
        refd = dy[a:b].float() @ w[e].float()
        assert (dx[a:b].float() - refd).abs().max().item() <= 2e-2 * refd.abs().max().item() + 1e-2
    # rows beyond the last group are left alone
    assert torch.isnan(y[offs[-1]:].float()).all()


@pytest.mark.parametrize("align", [128, 256])
@pytest.mark.parametrize("counts,M,N", [([130, 0, 257, 5], 768, 512), ([64, 700, 0], 256, 2048)])
def test_grouped_wgrad(counts, M, N, align):
    ops = ext.require()
    G = len(counts)
    offs_t, offs, R, valid = _layout(counts, align, extra_rows=64)
    g = torch.Generator(device="cuda").manual_seed(2)
    dy = torch.randn(R, M, device="cuda", generator=g).bfloat16() * valid[:, None]
    x = torch.randn(R, N, device="cuda", generator=g).bfloat16() * valid[:, None]
    dw = torch.full((G, M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped_bf16(dy, x, dw, offs_t, 2, align, False)
    torch.cuda.synchronize()
    assert ops.gemm_status(True) == 0
    for e in range(G):
        a, b = offs[e], offs[e + 1]
        ref = dy[a:b].float().t() @ x[a:b].float()
        assert (dw[e].float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("align", [128, 256])
def test_grouped_gemm_on_column_slices(align):
    """Row-indexed operands may be column halves of a wider buffer (strided rows): forward outputs written into the
    two halves of one [R, 2F] buffer, the halves read back as dgrad / wgrad operands, the second dgrad accumulated."""
    ops = ext.require()
    counts, F, D = [130, 0, 257, 5], 768, 512
    G = len(counts)
    offs_t, offs, R, valid = _layout(counts, align, extra_rows=align)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(R, D, device="cuda", generator=g).bfloat16() * valid[:, None]
    w1 = (torch.randn(G, F, D, device="cuda", generator=g) * 0.05).bfloat16()
    w3 = (torch.randn(G, F, D, device="cuda", generator=g) * 0.05).bfloat16()
    gu = torch.full((R, 2 * F), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped_bf16(x, w1, gu[:, :F], offs_t, 0, align, False)
    ops.gemm_grouped_bf16(x, w3, gu[:, F:], offs_t, 0, align, False)
    dgu = (torch.randn(R, 2 * F, device="cuda", generator=g) * valid[:, None]).bfloat16()
    dx = torch.full((R, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped_bf16(dgu[:, :F], w1, dx, offs_t, 1, align, False)
    ops.gemm_grouped_bf16(dgu[:, F:], w3, dx, offs_t, 1, align, True)
    dw3 = torch.full((G, F, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped_bf16(dgu[:, F:], x, dw3, offs_t, 2, align, False)
    torch.cuda.synchronize()
    assert ops.gemm_status(True) == 0
    for e in range(G):
        a, b = offs[e], offs[e + 1]
        if a == b:
            assert (dw3[e] == 0).all()
            continue
        for got, ref in ((gu[a:b, :F], x[a:b].float() @ w1[e].float().t()), (gu[a:b, F:], x[a:b].float() @ w3[e].float().t()),
                         (dx[a:b], dgu[a:b, :F].float() @ w1[e].float() + dgu[a:b, F:].float() @ w3[e].float()),
                         (dw3[e], dgu[a:b, F:].float().t() @ x[a:b].float())):
            assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 2e-2
    assert torch.isnan(gu[offs[-1]:].float()).all()
