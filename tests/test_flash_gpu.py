"""GPU: the tcgen05 flash-attention kernels against an fp32 dense-softmax reference."""

import math

import pytest
import torch

from torchtitan_b200.ops import ext

pytestmark = pytest.mark.gpu


def _reference(q, k, v, scale, causal, offset, kv_first):
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
    s = s.masked_fill(~mask[None], float("-inf"))
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


@pytest.mark.parametrize("Tq,Tk,Hq,Hkv,causal,offset,docs,packed", CASES)
def test_flash_forward(Tq, Tk, Hq, Hkv, causal, offset, docs, packed):
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
