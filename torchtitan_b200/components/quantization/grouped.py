"""Block-scaled fp8 numerics for the grouped (expert) GEMMs.

``quant_grouped_linear(x, w, offs, recipe, padded)`` is ``y[rows of e] = x[rows of e] @ w[e]^T`` with
both operands of each of the three GEMMs quantised along that GEMM's contraction dimension, like
:mod:`.linear` does for dense layers: forward along the input features, input gradient along the
output features, weight gradient along the tokens *of each expert*.  In the padded expert-major
layout every expert's rows start on a multiple of 128, so 32-row scale blocks never straddle two
experts and one column-wise quantiser call covers all experts; in the unpadded (sorted rows)
layout the token-axis quantisation runs per expert.

With ``mxfp8`` on a GPU, in the padded layout and with 128-multiple sizes, the three GEMMs run on
the block-scaled tensor-core kernel (``gemm_mxfp8_grouped``); otherwise on the operands' exact fp8
values held in bf16 (tcgen05 grouped GEMM on a GPU, PyTorch loops on CPU).  Parity: torchtitan/components/quantization/mx.py:104-206
(``MXFP8GroupedExpertsConverter``: torchao ``_quantize_then_scaled_grouped_mm``, recipe
``mxfp8_rceil``) and float8.py:216-266 (``Float8GroupedExpertsConverter``).
"""

from __future__ import annotations

import dataclasses

import torch

from .linear import fake_quant

__all__ = ["quant_grouped_linear", "quantize_experts"]


def _bounds(offs: torch.Tensor, padded: bool) -> list[tuple[int, int]]:
    o = [int(v) for v in offs.tolist()]
    if padded:       # offs[E + 1]: starts of the padded groups
        return [(o[i], o[i + 1]) for i in range(len(o) - 1)]
    return [(0 if i == 0 else o[i - 1], o[i]) for i in range(len(o))]   # cumulative ends


def _native(x: torch.Tensor, padded: bool) -> bool:
    from torchtitan_b200.ops import ext, functional as OF

    return padded and x.is_cuda and x.dtype == torch.bfloat16 and OF.settings.gemm == "tcgen05" and ext.available()


def _gemm(a, b, offs, mode, padded, out_shape):
    """mode 0: rows(e) @ b[e]^T; 1: rows(e) @ b[e]; 2: a_rows(e)^T @ b_rows(e) -> [E, N, K]."""
    out = torch.zeros(out_shape, dtype=a.dtype, device=a.device)
    if _native(a, padded):
        from torchtitan_b200.ops import moe_ops

        return moe_ops._gg(a.contiguous(), b.contiguous(), out, offs, mode)
    for e, (lo, hi) in enumerate(_bounds(offs, padded)):
        if hi <= lo:
            continue
        if mode == 0:
            out[lo:hi] = a[lo:hi] @ b[e].t()
        elif mode == 1:
            out[lo:hi] = a[lo:hi] @ b[e]
        else:
            out[e] = a[lo:hi].t() @ b[lo:hi]
    return out


def _fq_tokens(t: torch.Tensor, recipe: str, offs, padded: bool) -> torch.Tensor:
    """Quantise along the token axis inside each expert's row group."""
    if padded:
        return fake_quant(t.contiguous(), recipe, 0)
    out = torch.zeros_like(t)
    for lo, hi in _bounds(offs, padded):
        if hi > lo:
            out[lo:hi] = fake_quant(t[lo:hi].contiguous(), recipe, 0)
    return out


def _mx_native(x: torch.Tensor, w: torch.Tensor, recipe: str, padded: bool) -> bool:
    """The block-scaled grouped GEMM takes the padded layout and 128-multiples everywhere."""
    return (recipe == "mxfp8" and _native(x, padded) and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0
            and x.shape[0] % 128 == 0 and x.shape[0] > 0)


class _MXGroupedLinearFn(torch.autograd.Function):
    """All three grouped GEMMs on ``tcgen05.mma.kind::mxf8f6f4.block_scale`` (``gemm_mxfp8_grouped``)."""

    @staticmethod
    def forward(ctx, x, w, offs):
        from torchtitan_b200.ops import ext, functional as OF

        ops = ext.require()
        E, N, K = w.shape
        xq, xs = ops.mxfp8_quantize_tiled(x.contiguous())
        wq, ws = ops.mxfp8_quantize_tiled(w.reshape(E * N, K).contiguous())
        OF._count(3)
        ctx.save_for_backward(x, w, offs)
        return ops.gemm_mxfp8_grouped(xq, xs, wq, ws, offs, 1)

    @staticmethod
    def backward(ctx, dy):
        from torchtitan_b200.ops import ext, functional as OF

        ops = ext.require()
        x, w, offs = ctx.saved_tensors
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # contraction over the output features: every expert matrix transposed, then stacked [E K, N]
            gq, gs = ops.mxfp8_quantize_tiled(dy)
            wt = w.transpose(1, 2).contiguous().view(E * K, N)
            tq, ts = ops.mxfp8_quantize_tiled(wt)
            OF._count(3)
            dx = ops.gemm_mxfp8_grouped(gq, gs, tq, ts, offs, 1)
        if w.requires_grad:
            # contraction over each expert's tokens: both operands transposed by the quantiser
            gq, gs = ops.mxfp8_quantize_tiled_t(dy)
            xq, xs = ops.mxfp8_quantize_tiled_t(x.contiguous())
            OF._count(3)
            dw = OF._deliver_wgrad(w, ops.gemm_mxfp8_grouped(gq, gs, xq, xs, offs, 2).view(E, N, K))
        return dx, dw, None


class _QuantGroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offs, recipe, padded):
        E, N, K = w.shape
        xq = fake_quant(x.contiguous(), recipe, 1)
        wq = fake_quant(w.reshape(E * N, K).contiguous(), recipe, 1).view(E, N, K)
        ctx.save_for_backward(x, w, offs)
        ctx.recipe, ctx.padded = recipe, padded
        return _gemm(xq, wq, offs, 0, padded, (x.shape[0], N))

    @staticmethod
    def backward(ctx, dy):
        from torchtitan_b200.ops.functional import _deliver_wgrad

        x, w, offs = ctx.saved_tensors
        r, padded = ctx.recipe, ctx.padded
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # contraction over the output features: N % 32 == 0, so row blocks of the stacked [E N, K] stay inside an expert
            w_n = fake_quant(w.reshape(E * N, K).contiguous(), r, 0).view(E, N, K)
            dx = _gemm(fake_quant(dy, r, 1), w_n, offs, 1, padded, tuple(x.shape))
        if w.requires_grad:
            dw = _gemm(_fq_tokens(dy, r, offs, padded), _fq_tokens(x, r, offs, padded), offs, 2, padded, (E, N, K))
            dw = _deliver_wgrad(w, dw)
        return dx, dw, None, None, None


def quant_grouped_linear(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, recipe: str, padded: bool,
                         block_scaled: bool = True) -> torch.Tensor:
    if w.shape[1] % 32 or w.shape[2] % 32:
        raise ValueError("quantised grouped experts need feature dimensions that are multiples of 32")
    if block_scaled and _mx_native(x, w, recipe, padded):
        return _MXGroupedLinearFn.apply(x, w, offs)
    return _QuantGroupedLinearFn.apply(x, w, offs, recipe, padded)


def quantize_experts(model_cfg, recipe: str) -> int:
    """Config-tree rewrite: every ``GroupedExperts`` runs its three GEMMs with ``recipe`` numerics."""
    from torchtitan_b200.models.common.moe import GroupedExperts

    n = 0
    seen: set[int] = set()

    def walk(node):
        nonlocal n
        if id(node) in seen or not dataclasses.is_dataclass(node):
            return
        seen.add(id(node))
        if isinstance(node, GroupedExperts.Config):
            node.quant_recipe = recipe
            n += 1
        for f in dataclasses.fields(node):
            val = getattr(node, f.name, None)
            if dataclasses.is_dataclass(val):
                walk(val)
            elif isinstance(val, (list, tuple)):
                for item in val:
                    walk(item)

    walk(model_cfg)
    if n == 0:
        raise ValueError("the grouped-experts quantisation converter found no GroupedExperts in the model")
    return n
