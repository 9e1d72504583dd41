"""Optimizer-side flat kernels: AdamW on a shard, squared-norm accumulation, clip coefficient.

CUDA tensors use the sm_100a extension; CPU tensors use the PyTorch statement in
:mod:`reference`.  ``grad_scale`` may be a device scalar so that clipping needs no
host synchronisation.
"""

from __future__ import annotations

import torch

from . import ext, reference as ref
from .functional import _count

__all__ = ["adamw_", "sumsq_accumulate", "clip_coefficient"]


def adamw_(master, grad, exp_avg, exp_avg_sq, lowp_out, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    if master.numel() == 0:
        return
    if master.is_cuda:
        if not isinstance(grad_scale, torch.Tensor):
            grad_scale = torch.full((1,), float(grad_scale), dtype=torch.float32, device=master.device)
        bc1 = 1.0 - beta1 ** step
        bc2 = 1.0 - beta2 ** step
        _count()
        ext.require().adamw_(master, grad, exp_avg, exp_avg_sq, lowp_out, grad_scale.reshape(1),
                             float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
                             float(bc1), float(bc2))
        return
    ref.adamw_step(master, grad, exp_avg, exp_avg_sq, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                   weight_decay=weight_decay, step=step, grad_scale=grad_scale, out_lowp=lowp_out)


def sumsq_accumulate(x: torch.Tensor, acc: torch.Tensor) -> None:
    """``acc[0] += sum(x.float() ** 2)``."""
    if x.numel() == 0:
        return
    if x.is_cuda:
        _count()
        ext.require().sumsq_(x, acc)
        return
    acc.add_(x.float().pow(2).sum())


def clip_coefficient(total_norm: torch.Tensor, max_norm: float) -> torch.Tensor:
    """``min(1, max_norm / (norm + 1e-6))`` as a device scalar (torch.nn.utils.clip_grad_norm_ rule)."""
    return torch.clamp(max_norm / (total_norm + 1e-6), max=1.0)
