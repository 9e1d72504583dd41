"""GPU: the tcgen05 flash-attention kernels against an fp32 dense-softmax reference."""

import math

import pytest
import torch

from torchtitan_b200.ops import ext

pytestmark = pytest.mark.gpu


def _reference(q, k, v, scale, causal, offset, kv_first, window=0, sinks=None):
    """fp32 attention with explicit masks; returns (o [Tq,Hq,D], lse [Hq,Tq])."""
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    rows = torch.arange(Tq, device=q.device)[:, None]
    cols = torch.arange(Tk, device=q.device)[None, :]
    mask = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= cols <= rows + offset
    if kv_first is not None:
        mask &= cols >= kv_first.long()[:, None]
    if window:
        mask &= cols > rows + offset - window
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        s_ext = torch.cat([s, sinks.float()[:, None, None].expand(Hq, Tq, 1)], dim=-1)
        lse = torch.logsumexp(s_ext, dim=-1)
        p = torch.softmax(s_ext, dim=-1)[..., :-1]
    else:
        lse = torch.logsumexp(s, dim=-1)
        p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).transpose(0, 1), lse


def _inputs(Tq, Tk, Hq, Hkv, seed=0, packed=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    D = 128
    if packed and Tq == Tk:
        qkv = torch.randn(Tq, (Hq + 2 * Hkv) * D, device="cuda", generator=g).bfloat16()
        v3 = qkv.view(Tq, Hq + 2 * Hkv, D)
        return v3[:, :Hq], v3[:, Hq:Hq + Hkv], v3[:, Hq + Hkv:]
    q = torch.randn(Tq, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(Tk, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(Tk, Hkv, D, device="cuda", generator=g).bfloat16()
    return q, k, v


CASES = [
    # Tq, Tk, Hq, Hkv, causal, offset, docs, packed
    (128, 128, 2, 1, True, 0, False, False),
    (256, 256, 4, 2, True, 0, False, True),
    (1024, 1024, 8, 2, True, 0, False, True),
    (1000, 1000, 4, 4, True, 0, False, False),      # one head per CTA, ragged length
    (384, 640, 4, 2, False, 0, False, False),       # cross block, no mask
    (256, 512, 4, 2, True, 256, False, False),      # causal with offset (queries are the tail of the keys)
    (300, 556, 2, 1, False, 0, False, False),
    (1024, 1024, 4, 2, True, 0, True, True),        # packed documents
]


@pytest.fixture(params=[0, 1, 2, 3, 4], ids=lambda v: f"fwd{v}")
def fwd_variant(request):
    """Every forward kernel: 0 = whole-tile steps, 1..4 = the half-tile pipelined kernel (plain / packed fp32
    instructions / a quarter / a half of the exponentials on the FMA pipe)."""
    ops = ext.require()
    ops.flash_set_fwd_variant(request.param)
    yield request.param
    ops.flash_set_fwd_variant(0)


@pytest.mark.parametrize("Tq,Tk,Hq,Hkv,causal,offset,docs,packed", CASES)
def test_flash_forward(Tq, Tk, Hq, Hkv, causal, offset, docs, packed, fwd_variant):
    ops = ext.require()
    q, k, v = _inputs(Tq, Tk, Hq, Hkv, seed=Tq + Hq, packed=packed)
    kv_first = None
    if docs:
        starts = torch.tensor([0, 130, 131, 517, 900], device="cuda")
        pos = torch.arange(Tq, device="cuda")
        kv_first = starts[torch.searchsorted(starts, pos, right=True) - 1].int()
    scale = 1.0 / math.sqrt(128)
    o, lse = ops.flash_fwd(q, k, v, scale, causal, offset, kv_first)
    torch.cuda.synchronize()
    assert ops.flash_status(True) == 0
    o_ref, lse_ref = _reference(q, k, v, scale, causal, offset, kv_first)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref).abs().max().item() < 2e-2, (o.float() - o_ref).abs().max().item()
    assert (lse - lse_ref).abs().max().item() < 2e-2, (lse - lse_ref).abs().max().item()


@pytest.mark.parametrize("Tq,Tk,Hq,Hkv,causal,offset,docs,packed", CASES)
def test_flash_backward(Tq, Tk, Hq, Hkv, causal, offset, docs, packed):
    ops = ext.require()
    q, k, v = _inputs(Tq, Tk, Hq, Hkv, seed=Tq + Hq + 1, packed=packed)
    kv_first = None
    if docs:
        starts = torch.tensor([0, 130, 131, 517, 900], device="cuda")
        pos = torch.arange(Tq, device="cuda")
        kv_first = starts[torch.searchsorted(starts, pos, right=True) - 1].int()
    scale = 1.0 / math.sqrt(128)
    g = torch.Generator(device="cuda").manual_seed(7)
    d_o = torch.randn(Tq, Hq, 128, device="cuda", generator=g).bfloat16()
    o, lse = ops.flash_fwd(q, k, v, scale, causal, offset, kv_first)
    dq, dk, dv = ops.flash_bwd(d_o, q, k, v, o, lse, scale, causal, offset, kv_first, None, None, None)
    torch.cuda.synchronize()
    assert ops.flash_status(True) == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref, _ = _reference(qr, kr, vr, scale, causal, offset, kv_first)
    o_ref.backward(d_o.float())
    for name, got, ref in (("dq", dq, qr.grad), ("dk", dk, kr.grad), ("dv", dv, vr.grad)):
        err = (got.float() - ref).abs().max().item()
        tol = 2e-2 * ref.abs().max().item() + 2e-2
        assert err <= tol, (name, err, tol)


def test_flash_backward_into_packed_gradient():
    """dq / dk / dv written straight into slices of one packed [T, (Hq + 2 Hkv) * D] gradient."""
    ops = ext.require()
    T, Hq, Hkv, D = 512, 4, 2, 128
    q, k, v = _inputs(T, T, Hq, Hkv, seed=3, packed=True)
    scale = 1.0 / math.sqrt(D)
    d_o = torch.randn(T, Hq, D, device="cuda").bfloat16()
    o, lse = ops.flash_fwd(q, k, v, scale, True, 0, None)
    ref = ops.flash_bwd(d_o, q, k, v, o, lse, scale, True, 0, None, None, None, None)
    packed = torch.zeros(T, Hq + 2 * Hkv, D, device="cuda", dtype=torch.bfloat16)
    ops.flash_bwd(d_o, q, k, v, o, lse, scale, True, 0, None, packed[:, :Hq], packed[:, Hq:Hq + Hkv], packed[:, Hq + Hkv:])
    torch.cuda.synchronize()
    # dq is reduced across key blocks in no fixed order: equal up to fp32 summation order
    assert torch.allclose(packed[:, :Hq].float(), ref[0].float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(packed[:, Hq:Hq + Hkv], ref[1])
    assert torch.equal(packed[:, Hq + Hkv:], ref[2])


WINDOW_CASES = [
    # Tq, Tk, Hq, Hkv, offset, window, docs, sinks
    (1024, 1024, 4, 2, 0, 128, False, False),
    (1024, 1024, 4, 2, 0, 200, True, False),       # window and packed documents together
    (777, 777, 2, 2, 0, 64, False, True),          # ragged, one head per CTA, sinks
    (256, 768, 4, 2, 512, 300, False, False),      # queries are the tail of the keys
    (512, 512, 8, 2, 0, 0, False, True),           # sinks only
]


def _docs_kv_first(Tq):
    starts = torch.tensor([0, 130, 131, 517, 900], device="cuda")
    pos = torch.arange(Tq, device="cuda")
    return starts[torch.searchsorted(starts, pos, right=True) - 1].int()


@pytest.mark.parametrize("Tq,Tk,Hq,Hkv,offset,window,docs,use_sinks", WINDOW_CASES)
def test_flash_window_and_sinks(Tq, Tk, Hq, Hkv, offset, window, docs, use_sinks):
    """Sliding window and attention sinks, forward and backward, through the autograd front-end."""
    from torchtitan_b200.ops.flash import flash_attention_lse

    q, k, v = _inputs(Tq, Tk, Hq, Hkv, seed=Tq + window)
    kv_first = _docs_kv_first(Tq) if docs else None
    sinks = None
    if use_sinks:
        sinks = (torch.randn(Hq, device="cuda") * 2.0).requires_grad_()
    scale = 1.0 / math.sqrt(128)
    qg, kg, vg = (t.detach().clone().requires_grad_() for t in (q, k, v))
    o, lse = flash_attention_lse(qg, kg, vg, scale, causal=True, causal_offset=offset, kv_first=kv_first,
                                 window=window, sinks=sinks)
    d_o = torch.randn(Tq, Hq, 128, device="cuda").bfloat16()
    o.backward(d_o)
    torch.cuda.synchronize()
    assert ext.require().flash_status(True) == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    sr = sinks.detach().clone().requires_grad_() if use_sinks else None
    o_ref, lse_ref = _reference(qr, kr, vr, scale, True, offset, kv_first, window, sr)
    o_ref.backward(d_o.float())
    assert (o.float() - o_ref).abs().max().item() < 2e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2
    for name, got, ref in (("dq", qg.grad, qr.grad), ("dk", kg.grad, kr.grad), ("dv", vg.grad, vr.grad)):
        err = (got.float() - ref).abs().max().item()
        tol = 2e-2 * ref.abs().max().item() + 2e-2
        assert err <= tol, (name, err, tol)
    if use_sinks:
        err = (sinks.grad - sr.grad).abs().max().item()
        assert err <= 2e-2 * sr.grad.abs().max().item() + 2e-2, (err, sr.grad)


@pytest.mark.parametrize("D,window,use_sinks", [(64, 0, False), (64, 128, True), (16, 0, False), (96, 0, False)])
def test_small_head_dims_run_on_the_padded_kernels(D, window, use_sinks):
    """Head dimensions below 128 (GPT-OSS 64, debug models 16): zero-padded heads through the 128-wide kernels."""
    from torchtitan_b200.ops import functional as OF

    T, Hq, Hkv = 640, 4, 2
    g = torch.Generator(device="cuda").manual_seed(D)
    q = torch.randn(T, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(T, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(T, Hkv, D, device="cuda", generator=g).bfloat16()
    d_o = torch.randn(T, Hq, D, device="cuda", generator=g).bfloat16()
    sinks = torch.linspace(-1, 1, Hq, device="cuda").requires_grad_() if use_sinks else None
    scale = 1.0 / math.sqrt(D)
    before = OF.settings.library_fallbacks
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o = OF.attention(qg, kg, vg, scale=scale, causal=True, window=window or None, sinks=sinks)
    o.backward(d_o)
    assert OF.settings.library_fallbacks == before, "the call left the flash kernels"
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    sr = sinks.detach().clone().requires_grad_() if use_sinks else None
    o_ref, _ = _reference(qr, kr, vr, scale, True, 0, None, window, sr)
    o_ref.backward(d_o.float())
    assert o.shape == (T, Hq, D)
    assert (o.float() - o_ref).abs().max().item() < 2e-2
    for got, ref in ((qg.grad, qr.grad), (kg.grad, kr.grad), (vg.grad, vr.grad)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 2e-2
