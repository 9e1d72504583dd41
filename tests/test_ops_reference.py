"""CPU: the fused autograd functions agree with plain autograd over the same math."""

import math

import pytest
import torch
import torch.nn.functional as F

from torchtitan_b200.ops import functional as OF
from torchtitan_b200.ops import reference as ref

torch.manual_seed(0)


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def test_rms_norm_matches_autograd():
    x = torch.randn(12, 64, requires_grad=True)
    w = torch.randn(64, requires_grad=True)
    y = OF.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    y2 = _rms(x2, w2, 1e-5)
    y2.backward(g)
    assert torch.allclose(y, y2, atol=1e-6)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5)
    assert torch.allclose(w.grad, w2.grad, atol=1e-5)
    assert torch.allclose(y, F.rms_norm(x2, (64,), w2, 1e-5), atol=1e-6)


def test_norm_linear_and_swiglu_linear():
    x = torch.randn(10, 32, requires_grad=True)
    nw = torch.randn(32, requires_grad=True)
    W = torch.randn(48, 32, requires_grad=True)
    W2 = torch.randn(16, 24, requires_grad=True)
    gu = OF.norm_linear(x, nw, W, 1e-5)
    out = OF.swiglu_linear(gu, W2)
    g = torch.randn_like(out)
    out.backward(g)
    xs = [t.detach().clone().requires_grad_() for t in (x, nw, W, W2)]
    gu2 = _rms(xs[0], xs[1], 1e-5) @ xs[2].t()
    out2 = (F.silu(gu2[:, :24]) * gu2[:, 24:]) @ xs[3].t()
    out2.backward(g)
    assert torch.allclose(out, out2, atol=1e-5)
    for a, b in zip((x, nw, W, W2), xs):
        assert torch.allclose(a.grad, b.grad, atol=1e-4), (a.grad - b.grad).abs().max()


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_matches_complex_reference(interleaved):
    T, H, D = 7, 3, 16
    table = ref.rope_table(D, 32, 10000.0)
    pos = torch.randint(0, 32, (T,))
    x = torch.randn(T, H, D, requires_grad=True)
    y = OF.rope(x, table, pos, interleaved)
    ang = torch.outer(pos.float(), 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D)))
    if interleaved:
        xc = torch.view_as_complex(x.detach().reshape(T, H, D // 2, 2))
        exp = torch.view_as_real(xc * torch.polar(torch.ones_like(ang), ang)[:, None]).flatten(-2)
    else:
        cos, sin = torch.cat([ang, ang], -1).cos()[:, None], torch.cat([ang, ang], -1).sin()[:, None]
        xd = x.detach()
        rot = torch.cat([-xd[..., D // 2:], xd[..., :D // 2]], -1)
        exp = xd * cos + rot * sin
    assert torch.allclose(y, exp, atol=1e-5)
    # the backward is the inverse rotation: rope(grad) round trip
    g = torch.randn_like(y)
    y.backward(g)
    back = OF.rope(x.grad.detach(), table, pos, interleaved)
    assert torch.allclose(back, g, atol=1e-5)


def test_llama_rope_scaling_table():
    t = ref.rope_table(128, 16, 500000.0, "llama")
    t0 = ref.rope_table(128, 16, 500000.0, "none")
    # highest frequencies untouched, lowest divided by 8
    assert torch.allclose(t[:, 0], t0[:, 0])
    inv_low = 1.0 / (500000.0 ** (126 / 128))
    assert math.isclose(float(t[1, 64 + 63]), math.sin(inv_low / 8), rel_tol=1e-4)


def test_packed_rope_inplace():
    T, Hq, Hkv, D = 6, 4, 2, 8
    table = ref.rope_table(D, 16, 10000.0)
    pos = torch.arange(T)
    lin = torch.randn(T, (Hq + 2 * Hkv) * D, requires_grad=True)
    qkv = OF.rope_qk_(lin * 1.0, table, pos, True, Hq + Hkv, D).view(T, Hq + 2 * Hkv, D)
    exp_qk = ref.rope_apply(lin.detach().view(T, -1, D)[:, :Hq + Hkv], table, pos, True)
    assert torch.allclose(qkv[:, :Hq + Hkv], exp_qk, atol=1e-6)
    assert torch.equal(qkv[:, Hq + Hkv:], lin.detach().view(T, -1, D)[:, Hq + Hkv:])
    qkv.sum().backward()
    assert lin.grad is not None and torch.isfinite(lin.grad).all()


def test_linear_cross_entropy_matches_dense():
    T, Dm, V = 37, 16, 50
    h = torch.randn(T, Dm, requires_grad=True)
    W = torch.randn(V, Dm, requires_grad=True)
    labels = torch.randint(0, V, (T,))
    labels[::5] = -100
    n = (labels != -100).sum().float()
    loss = OF.linear_cross_entropy(h, W, labels, 1.0 / n, num_chunks=4)
    loss.backward()
    h2, W2 = h.detach().clone().requires_grad_(), W.detach().clone().requires_grad_()
    loss2 = F.cross_entropy(h2 @ W2.t(), labels, ignore_index=-100, reduction="sum") / n
    loss2.backward()
    assert torch.allclose(loss, loss2, atol=1e-5)
    assert torch.allclose(h.grad, h2.grad, atol=1e-5)
    assert torch.allclose(W.grad, W2.grad, atol=1e-5)


def test_cross_entropy_sum():
    logits = torch.randn(9, 11, requires_grad=True)
    labels = torch.randint(0, 11, (9,))
    labels[0] = -100
    loss = OF.cross_entropy_sum(logits, labels)
    loss.backward()
    l2 = logits.detach().clone().requires_grad_()
    F.cross_entropy(l2, labels, ignore_index=-100, reduction="sum").backward()
    assert torch.allclose(logits.grad, l2.grad, atol=1e-6)


def test_adamw_reference_matches_torch():
    p = torch.randn(100)
    g = torch.randn(100)
    master, m, v = p.clone(), torch.zeros(100), torch.zeros(100)
    tp = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([tp], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        tp.grad = g.clone()
        opt.step()
        ref.adamw_step(master, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    assert torch.allclose(master, tp.detach(), atol=1e-6)


def test_attention_document_mask():
    T, H, D = 10, 2, 8
    q, k, v = (torch.randn(T, H, D) for _ in range(3))
    doc = torch.tensor([1] * 4 + [2] * 6, dtype=torch.int32)
    out = OF.attention(q, k, v, doc_ids=doc)
    a = OF.attention(q[:4], k[:4], v[:4])
    b = OF.attention(q[4:], k[4:], v[4:])
    assert torch.allclose(out, torch.cat([a, b]), atol=1e-5)
    ref_out, _ = ref.attention_fwd(q, k, v, scale=1 / math.sqrt(D), doc_ids=doc)
    assert torch.allclose(out, ref_out, atol=1e-5)


def test_router_topk_counts():
    logits = torch.randn(20, 8)
    top, sel, counts = ref.router_topk(logits, 2, "softmax", None, True, 1.0)
    assert torch.allclose(top.sum(-1), torch.ones(20), atol=1e-5)
    assert counts.sum() == 40 and sel.shape == (20, 2)


def test_chunked_attention_fallback_matches_dense_autograd(monkeypatch):
    """The memory-bounded fallback (query blocks, probabilities recomputed in backward) against dense autograd math,
    with documents, a window, sinks and grouped heads; the block size is forced small so several blocks run."""
    import torch

    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.ops import reference as ref

    torch.manual_seed(0)
    T, Hq, Hkv, D = 70, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    doc = torch.tensor([0] * 20 + [1] * 33 + [2] * 17)
    sinks = torch.tensor([0.5, -1.0, 0.0, 2.0])
    g = torch.randn(T, Hq, D)
    monkeypatch.setattr(OF, "_DENSE_SCORE_BYTES", 4 * Hq * T * 16)     # 16 query rows per block
    a = [t.clone().requires_grad_() for t in (q, k, v, sinks)]
    out = OF._masked_attention(a[0], a[1], a[2], 0.3, True, doc, 9, a[3], None, None)
    out.backward(g)
    b = [t.clone().requires_grad_() for t in (q, k, v, sinks)]
    want, _ = ref.attention_fwd(b[0], b[1], b[2], scale=0.3, causal=True, doc_ids=doc, window=9, sinks=b[3])
    want.backward(g)
    assert torch.allclose(out, want, atol=1e-5)
    for x, y in zip(a, b):
        assert torch.allclose(x.grad, y.grad, atol=1e-4), (x.grad - y.grad).abs().max()
