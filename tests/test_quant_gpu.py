"""GPU: MXFP8 / float8 quantisation kernels against the PyTorch restatement of the same rounding."""

import pytest
import torch

from torchtitan_b200.ops import ext, reference as ref

pytestmark = pytest.mark.gpu


def _input(R, C, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(R, C, device="cuda", generator=g)
    x = x * torch.logspace(-4, 4, R, device="cuda")[:, None]   # many scale exponents
    x[0] = 0
    x[1, :32] = 448.0
    return x.bfloat16()


@pytest.mark.parametrize("R,C", [(64, 128), (100, 256), (513, 96)])
@pytest.mark.parametrize("axis", [0, 1])
def test_mxfp8_fake_quant_and_round_trip(R, C, axis):
    ops = ext.require()
    x = _input(R, C, seed=R + axis)
    fq = ops.mxfp8_fake_quant(x, axis)
    expect = ref.mxfp8_fake_quant(x.cpu(), axis).cuda()
    assert torch.equal(fq, expect)
    data, scales = ops.mxfp8_quantize(x, axis)
    assert data.shape == (R, C) and scales.shape == ((R, C // 32) if axis == 1 else ((R + 31) // 32, C))
    assert torch.equal(ops.mxfp8_dequantize(data, scales, axis), fq)
    # the stored bytes are e4m3 and e8m0 as torch understands them
    e = scales.view(torch.float8_e8m0fnu).float() if hasattr(torch, "float8_e8m0fnu") else torch.exp2(scales.float() - 127)
    vals = data.view(torch.float8_e4m3fn).float()
    full = e.repeat_interleave(32, dim=1) if axis == 1 else e.repeat_interleave(32, dim=0)[:R]
    assert torch.equal((vals * full).bfloat16(), fq)


def test_float8_rowwise():
    ops = ext.require()
    x = _input(200, 320, seed=3)
    fq = ops.float8_rowwise_fake_quant(x)
    expect = ref.float8_rowwise_fake_quant(x.cpu(), pow2=False).cuda()
    # same fp32 quotient on both sides; allow one e4m3 step in a vanishing fraction of elements
    row_max = expect.float().abs().amax(dim=1, keepdim=True)
    assert ((fq.float() - expect.float()).abs() <= row_max * 2 ** -3).all()
    assert (fq != expect).float().mean().item() < 1e-3
    data, scales = ops.float8_rowwise_quantize(x)
    assert torch.allclose((data.view(torch.float8_e4m3fn).float() * scales[:, None]).bfloat16().float(), fq.float())


def test_quant_linear_runs_on_gpu():
    from torchtitan_b200.components.quantization.linear import QuantLinear

    ext.require()
    lin = QuantLinear.Config(in_features=256, out_features=384, recipe="mxfp8").build()
    lin.init_states(seed=0)
    lin = lin.cuda().bfloat16()
    x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_()
    y = lin(x)
    y.backward(torch.randn_like(y))
    fq = ref.mxfp8_fake_quant
    want = fq(x.detach().cpu(), 1).float() @ fq(lin.weight.detach().cpu(), 1).float().t()
    assert (y.float().cpu() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-2
    assert x.grad is not None and lin.weight.grad is not None


def _untile(sf, R, K):
    """Tiled scale atoms -> [R, K/32] exponent bytes."""
    kt = K // 128
    a = sf.view((R + 127) // 128, kt, 32, 4, 4)          # [row tile, k tile, r % 32, r / 32, block]
    return a.permute(0, 3, 2, 1, 4).reshape(-1, kt * 4)[:R]


@pytest.mark.parametrize("R,C", [(128, 128), (300, 256), (1000, 384)])
def test_mxfp8_tiled_quantisers(R, C):
    ops = ext.require()
    x = _input(R, C, seed=R)
    data, scales = ops.mxfp8_quantize(x, 1)
    td, ts = ops.mxfp8_quantize_tiled(x)
    assert torch.equal(td, data) and torch.equal(_untile(ts, R, C), scales)
    # transposing form: x [Rt, Ct] scaled along its rows, written as [Ct, Rt]
    Rt, Ct = C, (R + 7) // 8 * 8
    xt = _input(Rt, Ct, seed=R + 1)
    d0, s0 = ops.mxfp8_quantize(xt, 0)                   # data [Rt, Ct], scales [Rt/32, Ct]
    dt, st = ops.mxfp8_quantize_tiled_t(xt)
    assert dt.shape == (Ct, Rt)
    assert torch.equal(dt, d0.t().contiguous()) and torch.equal(_untile(st, Ct, Rt), s0.t().contiguous())


@pytest.mark.parametrize("R,C", [(128, 128), (384, 256), (1024, 640)])
def test_mxfp8_dual_quantiser_equals_the_two_single_ones(R, C):
    """One read, both forms: row-wise and transposed outputs are bit-identical to the separate kernels."""
    ops = ext.require()
    x = _input(R, C, seed=R + C)
    d_row, s_row, d_t, s_t = ops.mxfp8_quantize_tiled_both(x)
    rd, rs = ops.mxfp8_quantize_tiled(x)
    td, ts = ops.mxfp8_quantize_tiled_t(x)
    assert torch.equal(d_row, rd) and torch.equal(s_row, rs)
    assert torch.equal(d_t, td) and torch.equal(s_t, ts)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (512, 256, 256), (1000, 520, 1024), (2048, 768, 512)])
def test_gemm_mxfp8_block_scaled(M, N, K, variant):
    ops = ext.require()
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 2, M, device="cuda")[:, None]).bfloat16()
    w = (torch.randn(N, K, device="cuda") * torch.logspace(-1, 1, N, device="cuda")[:, None]).bfloat16()
    xa, xs = ops.mxfp8_quantize_tiled(x)
    wa, ws = ops.mxfp8_quantize_tiled(w)
    ops.gemm_mx_set_variant(variant)
    try:
        c = ops.gemm_mxfp8(xa, xs, wa, ws)
        torch.cuda.synchronize()
    finally:
        ops.gemm_mx_set_variant(0)
    assert ops.gemm_status(True) == 0
    want = ops.mxfp8_fake_quant(x, 1).float() @ ops.mxfp8_fake_quant(w, 1).float().t()
    # bf16 rounding of the output, fp32 accumulation order
    err = (c.float() - want).abs()
    assert (err <= 1e-2 * want.abs() + 1e-3 * want.abs().max()).all(), err.max().item()


def test_float8_pow2_quantisers_match_reference():
    """Row-wise float8 with power-of-two scales in the block-scaled operand format: data and exponents against the
    PyTorch restatement, for both operand orientations."""
    ops = ext.require()
    x = _input(256, 384, seed=9)
    e_row = ref.float8_pow2_exponents(x.float().abs().amax(dim=1)).contiguous()
    d, s_ = ops.float8_pow2_quantize_tiled(x, e_row)
    scale = torch.exp2(e_row.float() - 127.0)[:, None]
    want = (x.float() / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(d.view(torch.float8_e4m3fn).float(), want.float())
    assert torch.equal(_untile(s_, 256, 384), e_row[:, None].expand(256, 384 // 32))
    e_col = ref.float8_pow2_exponents(x.float().abs().amax(dim=0)).contiguous()
    dt, st = ops.float8_pow2_quantize_tiled_t(x, e_col)
    scale_c = torch.exp2(e_col.float() - 127.0)[None, :]
    want_t = (x.float() / scale_c).clamp(-448, 448).to(torch.float8_e4m3fn).float().t()
    assert torch.equal(dt.view(torch.float8_e4m3fn).float(), want_t)
    assert torch.equal(_untile(st, 384, 256), e_col[:, None].expand(384, 256 // 32))


@pytest.mark.parametrize("recipe", ["mxfp8", "float8_rowwise"])
def test_quant_linear_block_scaled_matches_emulated(recipe):
    from torchtitan_b200.components.quantization.linear import QuantLinear

    ext.require()
    outs = []
    for block_scaled in (True, False):
        lin = QuantLinear.Config(in_features=256, out_features=384, recipe=recipe, block_scaled=block_scaled).build()
        lin.init_states(seed=0)
        lin = lin.cuda().bfloat16()
        g = torch.Generator(device="cuda").manual_seed(5)
        x = torch.randn(4, 128, 256, device="cuda", generator=g).bfloat16().requires_grad_()
        y = lin(x)
        y.backward(torch.randn(y.shape, device="cuda", generator=g).bfloat16())
        outs.append((y.detach().float(), x.grad.float(), lin.weight.grad.float()))
    for a, b in zip(*outs):
        assert (a - b).abs().max().item() <= 1e-2 * b.abs().max().item()


def test_quant_grouped_linear_padded_layout():
    """Expert GEMMs with MXFP8 numerics on the tcgen05 grouped GEMM against per-expert PyTorch."""
    from torchtitan_b200.components.quantization.grouped import quant_grouped_linear

    ext.require()
    torch.manual_seed(4)
    E, N, K = 3, 256, 128
    starts = [0, 256, 256, 640]            # padded groups (multiples of 128); expert 1 is empty
    offs = torch.tensor(starts, dtype=torch.int32, device="cuda")
    x = torch.randn(starts[-1], K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(E, N, K, device="cuda") * 0.1).bfloat16().requires_grad_()
    y = quant_grouped_linear(x, w, offs, "mxfp8", True)
    g = torch.randn_like(y)
    y.backward(g)
    fq = lambda t, a: ops_fq(t, a)
    ops_fq = ext.require().mxfp8_fake_quant
    for e in range(E):
        lo, hi = starts[e], starts[e + 1]
        if hi == lo:
            assert float(w.grad[e].abs().max()) == 0.0
            continue
        xe, ge, we = x.detach()[lo:hi].contiguous(), g[lo:hi].contiguous(), w.detach()[e].contiguous()
        want_y = fq(xe, 1).float() @ fq(we, 1).float().t()
        want_dx = fq(ge, 1).float() @ fq(we, 0).float()
        want_dw = fq(ge, 0).float().t() @ fq(xe, 0).float()
        for got, want in ((y[lo:hi], want_y), (x.grad[lo:hi], want_dx), (w.grad[e], want_dw)):
            assert (got.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3


def test_mx_grouped_linear_block_scaled_matches_emulated():
    """Grouped expert GEMMs on the block-scaled kernel against the emulated (exact fp8 in bf16) path."""
    from torchtitan_b200.components.quantization.grouped import quant_grouped_linear

    ext.require()
    torch.manual_seed(6)
    E, N, K = 4, 256, 384
    starts = [0, 128, 128, 512, 768]            # expert 1 is empty; 128 rows of tail padding
    R = 896
    offs = torch.tensor(starts, dtype=torch.int32, device="cuda")
    outs = []
    for block_scaled in (True, False):
        g = torch.Generator(device="cuda").manual_seed(9)
        x = torch.randn(R, K, device="cuda", generator=g).bfloat16()
        x[starts[-1]:] = 0
        x.requires_grad_()
        w = (torch.randn(E, N, K, device="cuda", generator=g) * 0.1).bfloat16().requires_grad_()
        y = quant_grouped_linear(x, w, offs, "mxfp8", True, block_scaled=block_scaled)
        gy = torch.randn(y.shape, device="cuda", generator=g).bfloat16()
        gy[starts[-1]:] = 0
        y.backward(gy)
        outs.append((y.detach().float()[:starts[-1]], x.grad.float()[:starts[-1]], w.grad.float()))
    assert ext.require().gemm_status(True) == 0
    for a, b in zip(*outs):
        assert (a - b).abs().max().item() <= 1e-2 * b.abs().max().item() + 1e-3
    assert float(outs[0][2][1].abs().max()) == 0.0      # the empty expert gets a zero gradient
