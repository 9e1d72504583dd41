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
    expect = ref.float8_rowwise_fake_quant(x.cpu()).cuda()
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
