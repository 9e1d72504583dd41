"""NVFP4 training linear: e2m1 elements, one e4m3 scale per 16 elements along the contraction
dimension, one fp32 scale per tensor.

Recipe (the NVFP4 v1 recipe of Transformer Engine / torchao that the reference wraps,
torchtitan/components/quantization/nvfp4.py:83-319):

* forward ``y = x w^T``: both operands rounded to nearest, blocks along the input features;
* input gradient ``dx = dy w``: ``dy`` with stochastic rounding, blocks along the output features;
* weight gradient ``dw = dy^T x``: both operands are first multiplied, along the token axis, by a
  16 x 16 random Hadamard transform (Sylvester matrix times a fixed sign vector, orthonormal, so
  it cancels in the product) that spreads outliers over their block; ``dy`` with stochastic
  rounding.  The sign vector is the same on every rank; the stochastic-rounding seed is a
  per-layer, per-rank buffer advanced every call.
* every GEMM dimension must be a multiple of 128; ``nvfp4_bf16_tail_fqns`` keeps the last
  fraction of the layers in bf16.

Execution: the quantiser is written with PyTorch tensor ops (it is the oracle and the
implementation; no hand-written kernel yet), the GEMMs run on the dequantised values on the bf16
tensor-core GEMM.  A ``kind::mxf4nvf4`` block-scaled GEMM is not built.
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass

import torch

from torchtitan_b200.models.common.layers import Linear
from torchtitan_b200.ops import functional as OF

__all__ = ["NVFP4Linear", "nvfp4_converter", "nvfp4_fake_quant", "nvfp4_bf16_tail_fqns", "hadamard16", "SIGN_VECTOR"]

SIGN_VECTOR = (1, 1, 1, -1, 1, -1, -1, -1, -1, -1, -1, 1, -1, 1, -1, -1)
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_BLOCK = 16
_DIM_MULTIPLE = 128


def hadamard16(device=None, dtype=torch.float32) -> torch.Tensor:
    """``diag(sign) . H16 / 4``: the orthonormal random Hadamard transform of the recipe."""
    h = torch.ones(1, 1)
    for _ in range(4):
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (torch.tensor(SIGN_VECTOR, dtype=torch.float32)[:, None] * h / 4.0).to(device=device, dtype=dtype)


def _round_e2m1(v: torch.Tensor, noise: torch.Tensor | None) -> torch.Tensor:
    """Magnitudes in [0, 6] -> e2m1 grid; nearest (ties to the even code) or stochastic."""
    grid = torch.tensor(_E2M1, device=v.device, dtype=v.dtype)
    hi_idx = torch.searchsorted(grid, v.clamp(max=6.0).contiguous(), right=False).clamp(max=7)
    lo_idx = (hi_idx - 1).clamp(min=0)
    lo, hi = grid[lo_idx], grid[hi_idx]
    span = (hi - lo).clamp_min(1e-30)
    frac = ((v - lo) / span).clamp(0, 1)
    if noise is not None:
        up = noise < frac
    else:
        up = (frac > 0.5) | ((frac == 0.5) & (hi_idx % 2 == 0))
    return torch.where(up | (hi_idx == lo_idx), hi, lo)


def nvfp4_fake_quant(x: torch.Tensor, axis: int, *, stochastic: bool = False, generator: torch.Generator | None = None,
                     rht: bool = False) -> torch.Tensor:
    """Values of ``x[R, C]`` after NVFP4 quantisation with 16-element blocks along ``axis``.

    With ``rht`` the transform is applied along ``axis`` first and the result stays in the
    transformed basis (both operands of a product over that axis are transformed, so it cancels)."""
    xt = (x if axis == 1 else x.t()).float()
    R, C = xt.shape
    if C % _BLOCK:
        raise ValueError(f"NVFP4 blocks need the contraction dimension ({C}) to be a multiple of {_BLOCK}")
    b = xt.reshape(R, C // _BLOCK, _BLOCK)
    if rht:
        b = b @ hadamard16(x.device)
    amax = b.abs().amax()
    gscale = torch.where(amax > 0, (448.0 * 6.0) / amax, torch.ones_like(amax))        # per-tensor, fp32
    bscale = (b.abs().amax(dim=-1, keepdim=True) / 6.0 * gscale).clamp(max=448.0)
    bscale = bscale.to(torch.float8_e4m3fn).float()                                    # per-block, e4m3
    denom = torch.where(bscale > 0, bscale / gscale, torch.ones_like(bscale))
    v = b / denom
    noise = None
    if stochastic:
        noise = torch.rand(v.shape, device=v.device, generator=generator)
    q = _round_e2m1(v.abs(), noise) * torch.sign(v)
    out = (q * denom).reshape(R, C)
    out = torch.where((bscale > 0).expand_as(b).reshape(R, C), out, torch.zeros_like(out))
    out = out if axis == 1 else out.t()
    return out.to(x.dtype).contiguous()


class _NVFP4LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, seed):
        x2 = x.reshape(-1, x.shape[-1])
        y = OF.gemm_nt(nvfp4_fake_quant(x2, 1), nvfp4_fake_quant(weight, 1))
        ctx.save_for_backward(x2, weight, seed)
        ctx.xshape = x.shape
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, seed = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        gen = torch.Generator(device=dy2.device)
        gen.manual_seed(int(seed.item()) & 0x7FFFFFFFFFFFFFFF)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = OF.gemm_nn(nvfp4_fake_quant(dy2, 1, stochastic=True, generator=gen),
                            nvfp4_fake_quant(weight, 0)).view(ctx.xshape)
        if weight.requires_grad:
            dw = OF._wgrad(nvfp4_fake_quant(dy2, 0, stochastic=True, generator=gen, rht=True),
                           nvfp4_fake_quant(x2, 0, rht=True), weight)
        return dx, dw, None


class NVFP4Linear(Linear):
    @dataclass(kw_only=True, slots=True)
    class Config(Linear.Config):
        pass

    def __init__(self, config: "NVFP4Linear.Config", **kw):
        super().__init__(config, **kw)
        for name in ("in_features", "out_features"):
            v = getattr(config, name)
            if v % _DIM_MULTIPLE:
                raise ValueError(f"NVFP4 requires {name} divisible by {_DIM_MULTIPLE}; got {v}: exclude this Linear "
                                 "from the converter's fqns")
        self._sr_seed: torch.Tensor | None = None   # per-rank runtime state, created on first use

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype != self.weight.dtype:
            x = x.to(self.weight.dtype)
        if x.reshape(-1, x.shape[-1]).shape[0] % _BLOCK:
            raise ValueError("NVFP4 needs the number of tokens to be a multiple of 16")
        if self._sr_seed is None or self._sr_seed.device != x.device:
            self._sr_seed = torch.randint(0, 2 ** 62, (1,), dtype=torch.int64, device=x.device)
        self._sr_seed += 1            # a fresh stochastic-rounding stream every call
        y = _NVFP4LinearFn.apply(x, self.weight, self._sr_seed.clone())
        return y if self.bias is None else y + self.bias


def nvfp4_bf16_tail_fqns(num_layers: int, bf16_tail_fraction: float) -> list[str]:
    """FQN filters that convert the leading layers and keep the last
    ``ceil(num_layers * fraction)`` in bf16 (``layers.1.`` does not match ``layers.10``)."""
    upto = num_layers - math.ceil(num_layers * bf16_tail_fraction)
    if upto <= 0:
        raise ValueError(f"bf16_tail_fraction={bf16_tail_fraction} keeps all {num_layers} layers in bf16")
    return [f"layers.{i}." for i in range(upto)]


def nvfp4_converter(model_cfg, arg, job_config) -> int:
    """``arg``: comma-separated FQN substrings (default: every attention / MLP linear), or
    ``tail=<fraction>`` to keep the last fraction of the layers in bf16."""
    from .utils import iter_linear_configs, module_filter

    opts = [a for a in (arg or "").split(",") if a]
    fqns: list[str] = []
    for o in opts:
        if o.startswith("tail="):
            fqns += nvfp4_bf16_tail_fqns(len(model_cfg.layers), float(o[5:]))
        else:
            fqns.append(o)
    n = 0
    for fqn, owner, attr, lin in list(iter_linear_configs(model_cfg)):
        if type(lin).__qualname__ != "Linear.Config" or not module_filter(fqn, lin, fqns or None):
            continue
        kw = {f.name: getattr(lin, f.name) for f in dataclasses.fields(lin)}
        setattr(owner, attr, NVFP4Linear.Config(**kw))
        n += 1
    if n == 0:
        raise ValueError("the NVFP4 converter matched no Linear layer")
    return n
