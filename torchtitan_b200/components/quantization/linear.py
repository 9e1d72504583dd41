"""Linear layers whose three GEMMs run on block-scaled fp8 operands.

Recipes.  ``mxfp8``: each GEMM quantises both operands to MXFP8 (e4m3 elements, one e8m0 scale
per 32 elements *along that GEMM's contraction dimension*, RCEIL scale rounding): the forward
scales ``x`` and ``w`` along the input features, the input gradient scales ``dy`` along the
output features and ``w`` along its rows, the weight gradient scales ``dy`` and ``x`` along the
tokens.  Outputs and accumulation stay bf16 / fp32.  ``float8_rowwise``: one fp32 scale per row of
each operand (e4m3).  Parity: torchao ``MXFP8Linear`` / row-wise ``Float8Linear`` as configured
by torchtitan/components/quantization/mx.py:50-98 and float8.py:53-173.

Execution.  The quantisers are hand-written kernels (``ops/csrc/quant.cu``).  With the ``mxfp8``
recipe on a GPU, every GEMM whose contraction dimension is a multiple of 128 runs on the
block-scaled tensor-core path (``ops/csrc/gemm_mx.cu``: ``tcgen05.mma.kind::mxf8f6f4.block_scale``
on e4m3 bytes and e8m0 scales; the operands that are contracted over their rows are quantised by a
transposing kernel so that both arrive K-major).  Otherwise, and for ``float8_rowwise``, the GEMM
runs on the operands' *exact* fp8 values held in bf16 (every e4m3 x 2^e product is representable
in bf16) on the tcgen05 bf16 GEMM with fp32 accumulation: the same numerics at bf16 throughput.
``float8_rowwise`` uses power-of-two row scales (the reference recipe's ``round_scales_to_power_of_2``), which are
e8m0 scales that are equal along a row: on a GPU its GEMMs therefore run on the same block-scaled kernel, with the
quantisers taking the per-row exponents as an input (``float8_pow2_quantize_tiled`` / ``_t``).
On CPU the same math runs in PyTorch (``ops.reference``), which is also the oracle of the kernel
tests.  ``block_scaled = False`` in the layer's config forces the emulated path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from torchtitan_b200.models.common.layers import Linear
from torchtitan_b200.ops import ext, functional as OF, reference as ref

__all__ = ["QuantLinear", "fake_quant"]


def fake_quant(x: torch.Tensor, recipe: str, axis: int) -> torch.Tensor:
    """Values of ``x[R, C]`` after a round trip through the recipe's fp8 format, scaled along ``axis``."""
    if recipe == "mxfp8":
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and (axis == 0 or x.shape[1] % 32 == 0):
            OF._count()
            return ext.require().mxfp8_fake_quant(x.contiguous(), axis)
        return ref.mxfp8_fake_quant(x, axis)
    if recipe == "float8_rowwise":
        xt = x if axis == 1 else x.t()
        out = ref.float8_rowwise_fake_quant(xt)      # power-of-two row scales (tensor ops; the emulated path only)
        return out if axis == 1 else out.t()
    raise ValueError(f"unknown quantisation recipe '{recipe}'")


def _mx_native(recipe: str, block_scaled: bool, contraction: int, n_out: int, *ts: torch.Tensor) -> bool:
    """Whether a GEMM can run on the block-scaled tensor-core kernel."""
    return (block_scaled and recipe == "mxfp8" and contraction > 0 and contraction % 128 == 0 and n_out % 8 == 0
            and all(t.is_cuda and t.dtype == torch.bfloat16 and t.shape[1] % 8 == 0 for t in ts) and ext.available())


def _mx_gemm(a: torch.Tensor, a_rows_contracted: bool, b: torch.Tensor, b_rows_contracted: bool) -> torch.Tensor:
    """Block-scaled GEMM of two bf16 operands, each quantised along its contraction dimension.

    An operand given as [contraction, rows] (``*_rows_contracted``) goes through the transposing
    quantiser; the result is ``A_q [M, K] . B_q [N, K]^T`` in bf16."""
    ops = ext.require()
    OF._count(3)
    qa = ops.mxfp8_quantize_tiled_t(a) if a_rows_contracted else ops.mxfp8_quantize_tiled(a)
    qb = ops.mxfp8_quantize_tiled_t(b) if b_rows_contracted else ops.mxfp8_quantize_tiled(b)
    return ops.gemm_mxfp8(qa[0], qa[1], qb[0], qb[1])


def _f8_native(recipe: str, block_scaled: bool, contraction: int, n_out: int, *ts: torch.Tensor) -> bool:
    """Whether a float8 row-wise GEMM can run on the block-scaled tensor-core kernel (power-of-two row scales are
    e8m0 scales that happen to be equal along a row)."""
    return (block_scaled and recipe == "float8_rowwise" and contraction > 0 and contraction % 128 == 0 and n_out % 8 == 0
            and all(t.is_cuda and t.dtype == torch.bfloat16 and t.shape[1] % 8 == 0 for t in ts) and ext.available())


def _f8_operand(t: torch.Tensor, rows_contracted: bool):
    """Quantise ``t`` for a float8 row-wise GEMM: one power-of-two scale per output row, i.e. per row of ``t`` when it
    is given as [rows, contraction] and per column when it is given as [contraction, rows]."""
    ops = ext.require()
    OF._count(2)
    if rows_contracted:
        exps = ref.float8_pow2_exponents(t.abs().amax(dim=0))
        return ops.float8_pow2_quantize_tiled_t(t, exps.contiguous())
    exps = ref.float8_pow2_exponents(t.abs().amax(dim=1))
    return ops.float8_pow2_quantize_tiled(t, exps.contiguous())


def _f8_gemm(a: torch.Tensor, a_rows_contracted: bool, b: torch.Tensor, b_rows_contracted: bool) -> torch.Tensor:
    qa, qb = _f8_operand(a, a_rows_contracted), _f8_operand(b, b_rows_contracted)
    OF._count()
    return ext.require().gemm_mxfp8(qa[0], qa[1], qb[0], qb[1])


def _both_ok(t: torch.Tensor) -> bool:
    return t.shape[0] % 128 == 0 and t.shape[1] % 128 == 0


class _QuantLinearFn(torch.autograd.Function):
    """``y = x w^T`` with all three GEMMs on quantised operands.  On the block-scaled path an operand that two GEMMs
    contract over different dimensions (``x``: features in the forward, tokens in the weight gradient; ``dy``:
    output features in the input gradient, tokens in the weight gradient) is quantised in both forms by one kernel
    from one read; the forward then keeps the transposed fp8 form of ``x`` for the backward instead of bf16 ``x``."""

    @staticmethod
    def forward(ctx, x, weight, recipe, hp_wgrad, block_scaled=True):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.x_t = None
        saved_x = x2
        if _mx_native(recipe, block_scaled, x2.shape[1], weight.shape[0], x2, weight):
            ops = ext.require()
            wgrad_native = (weight.requires_grad and not hp_wgrad and _both_ok(x2)
                            and _mx_native(recipe, block_scaled, x2.shape[0], weight.shape[1], x2))
            qw = ops.mxfp8_quantize_tiled(weight)
            if wgrad_native:
                qx = ops.mxfp8_quantize_tiled_both(x2)
                ctx.x_t = (qx[2], qx[3])          # [features, tokens] fp8 + scales: the weight gradient's operand
                saved_x = x2.new_empty(0)
                OF._count(3)
            else:
                qx = ops.mxfp8_quantize_tiled(x2)
                OF._count(3)
            y = ops.gemm_mxfp8(qx[0], qx[1], qw[0], qw[1])
        elif _f8_native(recipe, block_scaled, x2.shape[1], weight.shape[0], x2, weight):
            y = _f8_gemm(x2, False, weight, False)
        else:
            y = OF.gemm_nt(fake_quant(x2, recipe, 1), fake_quant(weight, recipe, 1))
        ctx.save_for_backward(saved_x, weight)
        ctx.recipe, ctx.hp_wgrad, ctx.xshape, ctx.block_scaled = recipe, hp_wgrad, x.shape, block_scaled
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        r = ctx.recipe
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        bs = ctx.block_scaled
        ops = ext.require() if dy2.is_cuda else None
        x_t = ctx.x_t
        ctx.x_t = None
        need_dx = ctx.needs_input_grad[0]
        dgrad_native = need_dx and _mx_native(r, bs, weight.shape[0], weight.shape[1], dy2, weight)
        wgrad_native = weight.requires_grad and not ctx.hp_wgrad and x_t is not None
        q_dy = None
        if dgrad_native and wgrad_native and _both_ok(dy2):
            q_dy = ops.mxfp8_quantize_tiled_both(dy2)     # one read of dy for both gradients
            OF._count()
        if need_dx:
            # contraction over the output features: dy along its columns, w along its rows
            if dgrad_native:
                qa = (q_dy[0], q_dy[1]) if q_dy is not None else ops.mxfp8_quantize_tiled(dy2)
                qb = ops.mxfp8_quantize_tiled_t(weight)
                OF._count(3)
                dx = ops.gemm_mxfp8(qa[0], qa[1], qb[0], qb[1]).view(ctx.xshape)
            elif _f8_native(r, bs, weight.shape[0], weight.shape[1], dy2, weight):
                dx = _f8_gemm(dy2, False, weight, True).view(ctx.xshape)
            else:
                dx = OF.gemm_nn(fake_quant(dy2, r, 1), fake_quant(weight, r, 0)).view(ctx.xshape)
        dw = None
        if weight.requires_grad:
            if ctx.hp_wgrad:
                dw = OF._wgrad(dy2, x2, weight)
            elif wgrad_native:                                            # contraction over the tokens
                qa = (q_dy[2], q_dy[3]) if q_dy is not None else ops.mxfp8_quantize_tiled_t(dy2)
                OF._count(2)
                dw = OF._deliver_wgrad(weight, ops.gemm_mxfp8(qa[0], qa[1], x_t[0], x_t[1]))
            elif _mx_native(r, bs, dy2.shape[0], weight.shape[1], dy2, x2):
                dw = OF._deliver_wgrad(weight, _mx_gemm(dy2, True, x2, True))
            elif _f8_native(r, bs, dy2.shape[0], weight.shape[1], dy2, x2):
                dw = OF._deliver_wgrad(weight, _f8_gemm(dy2, True, x2, True))
            else:
                dw = OF._wgrad(fake_quant(dy2, r, 0), fake_quant(x2, r, 0), weight)
        return dx, dw, None, None, None


class QuantLinear(Linear):
    @dataclass(kw_only=True, slots=True)
    class Config(Linear.Config):
        recipe: str = "mxfp8"  # "mxfp8" | "float8_rowwise"
        high_precision_wgrad: bool = False  # rowwise_with_gw_hp of the float8 recipe
        block_scaled: bool = True  # mxfp8 on a GPU: run the GEMMs on the block-scaled tensor-core kernel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        if x.dtype != self.weight.dtype:
            x = x.to(self.weight.dtype)
        y = _QuantLinearFn.apply(x, self.weight, c.recipe, c.high_precision_wgrad, c.block_scaled)
        return y if self.bias is None else y + self.bias
