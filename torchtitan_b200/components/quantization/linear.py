"""Linear layers whose three GEMMs run on block-scaled fp8 operands.

Recipes.  ``mxfp8``: each GEMM quantises both operands to MXFP8 (e4m3 elements, one e8m0 scale
per 32 elements *along that GEMM's contraction dimension*, RCEIL scale rounding): the forward
scales ``x`` and ``w`` along the input features, the input gradient scales ``dy`` along the
output features and ``w`` along its rows, the weight gradient scales ``dy`` and ``x`` along the
tokens.  Outputs and accumulation stay bf16 / fp32.  ``float8_rowwise``: one fp32 scale per row of
each operand (e4m3).  Parity: torchao ``MXFP8Linear`` / row-wise ``Float8Linear`` as configured
by torchtitan/components/quantization/mx.py:50-98 and float8.py:53-173.

Execution.  The quantiser is a hand-written kernel (``ops/csrc/quant.cu``).  The GEMM itself runs
on the operands' *exact* MXFP8 values in bf16 (every e4m3 x 2^e product is representable in
bf16), on the tcgen05 bf16 GEMM with fp32 accumulation, so the numerics are those of a
block-scaled fp8 GEMM while the throughput is that of bf16.  On CPU the same math runs in
PyTorch (``ops.reference``), which is also the oracle of the kernel tests.
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
        if x.is_cuda and x.dtype == torch.bfloat16 and xt.shape[1] % 8 == 0:
            OF._count()
            out = ext.require().float8_rowwise_fake_quant(xt.contiguous())
        else:
            out = ref.float8_rowwise_fake_quant(xt)
        return out if axis == 1 else out.t()
    raise ValueError(f"unknown quantisation recipe '{recipe}'")


class _QuantLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, recipe, hp_wgrad):
        x2 = x.reshape(-1, x.shape[-1])
        y = OF.gemm_nt(fake_quant(x2, recipe, 1), fake_quant(weight, recipe, 1))
        ctx.save_for_backward(x2, weight)
        ctx.recipe, ctx.hp_wgrad, ctx.xshape = recipe, hp_wgrad, x.shape
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        r = ctx.recipe
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            # contraction over the output features: dy along its columns, w along its rows
            dx = OF.gemm_nn(fake_quant(dy2, r, 1), fake_quant(weight, r, 0)).view(ctx.xshape)
        dw = None
        if weight.requires_grad:
            if ctx.hp_wgrad:
                dw = OF._wgrad(dy2, x2, weight)
            else:  # contraction over the tokens
                dw = OF._wgrad(fake_quant(dy2, r, 0), fake_quant(x2, r, 0), weight)
        return dx, dw, None, None


class QuantLinear(Linear):
    @dataclass(kw_only=True, slots=True)
    class Config(Linear.Config):
        recipe: str = "mxfp8"  # "mxfp8" | "float8_rowwise"
        high_precision_wgrad: bool = False  # rowwise_with_gw_hp of the float8 recipe

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        if x.dtype != self.weight.dtype:
            x = x.to(self.weight.dtype)
        y = _QuantLinearFn.apply(x, self.weight, c.recipe, c.high_precision_wgrad)
        return y if self.bias is None else y + self.bias
