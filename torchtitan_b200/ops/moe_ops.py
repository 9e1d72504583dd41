"""Autograd front-ends of the MoE kernels: router, padded expert-major permute, grouped expert
GEMMs (tcgen05) and the weighted combine.

Layout.  After routing, slot ``(t, k)`` (token ``t``, k-th choice) is assigned row
``dest[t, k]`` of an expert-major buffer in which every expert's rows start at a multiple of
``ALIGN`` rows (128): no GEMM tile straddles two experts and the weight-gradient K loop of an
expert starts on a tile boundary.  Padding rows are zero.  The buffer has the static capacity
``T*K + E*(ALIGN-1)`` rounded up, so no host synchronisation is needed to size it.
(The reference pads groups the same way for its quantised grouped GEMMs,
torchtitan/models/common/token_dispatcher.py:733-775, and calls ``torch._grouped_mm``.)
"""

from __future__ import annotations

import torch

from . import ext
from .functional import _count, _deliver_wgrad

ALIGN = 128

__all__ = ["ALIGN", "router_topk", "padded_layout", "permute_rows", "combine_rows", "gather_rows", "grouped_linear",
           "grouped_swiglu_experts", "native_ok"]


def native_ok(x: torch.Tensor, dim: int, hidden: int) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and dim % 64 == 0 and hidden % 128 == 0 and ext.available()


# ---------------------------------------------------------------------------------------------
class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, top_k, sigmoid, route_norm, route_scale):
        ops = ext.require()
        logits = logits.contiguous()
        top, sel, counts = ops.moe_router_fwd(logits, bias, top_k, sigmoid, route_norm, route_scale)
        _count()
        ctx.save_for_backward(logits, sel)
        ctx.meta = (sigmoid, route_norm, route_scale)
        ctx.mark_non_differentiable(sel, counts)
        return top, sel, counts

    @staticmethod
    def backward(ctx, dtop, _dsel, _dcounts):
        logits, sel = ctx.saved_tensors
        sigmoid, route_norm, route_scale = ctx.meta
        _count()
        dl = ext.require().moe_router_bwd(logits, sel, dtop.contiguous().float(), sigmoid, route_norm, route_scale)
        return dl, None, None, None, None, None


def router_topk(logits: torch.Tensor, bias: torch.Tensor | None, top_k: int, score_func: str, route_norm: bool,
                route_scale: float):
    """fp32 gate logits ``[T, E]`` -> (scores of the chosen experts ``[T, K]`` fp32 with gradient,
    chosen experts ``[T, K]`` int32, tokens per expert ``[E]`` fp32)."""
    return _RouterFn.apply(logits, bias, int(top_k), score_func == "sigmoid", bool(route_norm), float(route_scale))


def padded_layout(selected: torch.Tensor, counts: torch.Tensor, align: int = ALIGN):
    """``selected[T, K]`` expert ids, ``counts[E]`` -> (``dest[T, K]`` int32 rows of the padded
    expert-major buffer, ``offs[E + 1]`` int32 group starts, static row capacity).  Rows of one
    expert keep token order (stable), so results do not depend on scheduling."""
    T, K = selected.shape
    E = counts.numel()
    flat = selected.reshape(-1).long()
    c = counts.to(torch.int64)
    padded = (c + (align - 1)) // align * align
    offs = torch.zeros(E + 1, dtype=torch.int64, device=selected.device)
    offs[1:] = torch.cumsum(padded, 0)
    start = torch.cumsum(c, 0) - c
    order = torch.argsort(flat, stable=True)
    e_sorted = flat[order]
    pos_in_expert = torch.arange(T * K, device=selected.device) - start[e_sorted]
    dest = torch.empty(T * K, dtype=torch.int64, device=selected.device)
    dest[order] = offs[e_sorted] + pos_in_expert
    cap = (T * K + E * (align - 1) + align - 1) // align * align
    return dest.view(T, K).to(torch.int32), offs.to(torch.int32), cap


class _PermuteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, rows):
        ctx.save_for_backward(dest)
        _count()
        return ext.require().moe_permute_rows(x.contiguous(), dest, rows)

    @staticmethod
    def backward(ctx, dy):
        (dest,) = ctx.saved_tensors
        _count()
        return ext.require().moe_combine_rows(dy.contiguous(), dest, None), None, None


def permute_rows(x: torch.Tensor, dest: torch.Tensor, rows: int) -> torch.Tensor:
    return _PermuteFn.apply(x, dest, rows)


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, dest):
        ctx.save_for_backward(dest)
        ctx.rows = y.shape[0]
        _count()
        return ext.require().moe_combine_rows(y.contiguous(), dest, None)

    @staticmethod
    def backward(ctx, dout):
        (dest,) = ctx.saved_tensors
        _count()
        return ext.require().moe_permute_rows(dout.contiguous(), dest, ctx.rows), None


def gather_rows(y: torch.Tensor, dest: torch.Tensor) -> torch.Tensor:
    """``out[i] = sum_k y[dest[i, k]]`` (``K = 1``: a plain row gather); inverse of ``permute_rows``."""
    return _GatherFn.apply(y, dest)


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, dest, wts):
        wts = wts.contiguous().float()
        ctx.save_for_backward(y, dest, wts)
        _count()
        return ext.require().moe_combine_rows(y, dest, wts)

    @staticmethod
    def backward(ctx, dout):
        y, dest, wts = ctx.saved_tensors
        _count()
        dy, dw = ext.require().moe_combine_bwd(dout.contiguous(), y, dest, wts)
        return dy, None, dw


def combine_rows(y: torch.Tensor, dest: torch.Tensor, wts: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_k wts[t, k] * y[dest[t, k]]`` (fp32 accumulation, bf16 result)."""
    return _CombineFn.apply(y.contiguous(), dest, wts)


# ---------------------------------------------------------------------------------------------
def _gg(a, b, c, offs, mode, accumulate=False):
    _count()
    ext.require().gemm_grouped_bf16(a, b, c, offs, mode, ALIGN, accumulate)
    return c


class _GroupedLinearFn(torch.autograd.Function):
    """``y[rows of e] = x[rows of e] @ w[e]^T`` with ``w[E, N, K]``."""

    @staticmethod
    def forward(ctx, x, w, offs):
        y = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        _gg(x, w, y, offs, 0)
        ctx.save_for_backward(x, w, offs)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, offs = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _gg(dy, w, dx, offs, 1)
        dw = None
        if w.requires_grad:
            dw = _grouped_wgrad(dy, x, w, offs)
        return dx, dw, None


def _grouped_wgrad(dy, x, w, offs):
    mg = getattr(w, "main_grad", None)
    if mg is not None and mg.dtype == dy.dtype:
        acc = getattr(w, "_main_grad_written", False)
        _gg(dy, x, mg.view(w.shape), offs, 2, accumulate=acc)
        w._main_grad_written = True
        return None
    dw = torch.empty(w.shape, dtype=dy.dtype, device=dy.device)
    _gg(dy, x, dw, offs, 2)
    return _deliver_wgrad(w, dw)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    return _GroupedLinearFn.apply(x, w, offs)


def swiglu_experts_fwd(x, w1, w3, w2, offs, out=None):
    """``(silu(x w1^T) * (x w3^T)) w2^T`` per expert on the padded layout; returns ``(y, gu)`` with ``gu[R, 2F]`` the
    two first GEMM outputs side by side (what the backward keeps).  ``out``: write ``y`` into this buffer."""
    R = x.shape[0]
    F_ = w1.shape[1]
    # the two projections write the column halves of one [R, 2F] buffer (strided output rows), the layout the
    # SwiGLU kernel takes
    gu = torch.empty(R, 2 * F_, dtype=x.dtype, device=x.device)
    _gg(x, w1, gu[:, :F_], offs, 0)
    _gg(x, w3, gu[:, F_:], offs, 0)
    # rows at or beyond offs[-1] hold whatever the allocator returned; they are never consumed
    a = ext.require().swiglu_fwd(gu)
    _count()
    y = out if out is not None else torch.empty(R, w2.shape[1], dtype=x.dtype, device=x.device)
    _gg(a, w2, y, offs, 0)
    return y, gu


def swiglu_experts_bwd(dy, x, gu, w1, w3, w2, offs, need_dx=True, dx_out=None):
    """Backward of :func:`swiglu_experts_fwd`: the activation is recomputed from ``gu``; weight gradients go to the
    parameters' ``main_grad`` buffers when they have them (then the returned ``dw`` is None).  ``dx_out``: write the
    input gradient into this buffer.  Returns ``(dx, dw1, dw3, dw2)``."""
    ops = ext.require()
    dy = dy.contiguous()
    F_ = w1.shape[1]
    a = ops.swiglu_fwd(gu)
    dw2 = _grouped_wgrad(dy, a, w2, offs) if w2.requires_grad else None
    # rows at or beyond offs[-1] of da / dgu / dx are never written nor consumed (the grouped GEMMs only visit
    # the padded groups), so none of these buffers needs clearing
    da = torch.empty_like(a)
    del a
    _gg(dy, w2, da, offs, 1)
    dgu = ops.swiglu_bwd(gu, da)
    _count(2)
    del da
    dh, du = dgu[:, :F_], dgu[:, F_:]        # column halves, read in place through strided tensor maps
    dw1 = _grouped_wgrad(dh, x, w1, offs) if w1.requires_grad else None
    dw3 = _grouped_wgrad(du, x, w3, offs) if w3.requires_grad else None
    dx = None
    if need_dx:
        dx = dx_out if dx_out is not None else torch.empty_like(x)
        _gg(dh, w1, dx, offs, 1)
        _gg(du, w3, dx, offs, 1, accumulate=True)
    return dx, dw1, dw3, dw2


class _GroupedSwiGLUExpertsFn(torch.autograd.Function):
    """Autograd form of ``swiglu_experts_fwd`` / ``swiglu_experts_bwd``, keeping ``x`` and ``gu``; the activation is
    recomputed in backward (same policy as the dense SwiGLU MLP)."""

    @staticmethod
    def forward(ctx, x, w1, w3, w2, offs):
        y, gu = swiglu_experts_fwd(x, w1, w3, w2, offs)
        ctx.save_for_backward(x, gu, w1, w3, w2, offs)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gu, w1, w3, w2, offs = ctx.saved_tensors
        dx, dw1, dw3, dw2 = swiglu_experts_bwd(dy, x, gu, w1, w3, w2, offs, need_dx=ctx.needs_input_grad[0])
        return dx, dw1, dw3, dw2, None


def grouped_swiglu_experts(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor,
                           offs: torch.Tensor) -> torch.Tensor:
    """``x[R, D]`` in the padded expert-major layout, ``w1/w3[E, F, D]``, ``w2[E, D, F]``."""
    return _GroupedSwiGLUExpertsFn.apply(x, w1, w3, w2, offs)
