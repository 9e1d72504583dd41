"""Autograd-aware collectives for tensor / sequence parallelism.

Each function takes a ``TPContext``-like object (``group``, ``size``, ``rank``).
Forward/backward duals follow the placement contracts of the reference
(torchtitan/models/common/decoder_sharding.py:121-338):

========================  =======================  =========================
function                  forward                  backward
========================  =======================  =========================
``all_gather_rows``       S(0) -> R  (all-gather)  P -> S(0) (reduce-scatter)
``reduce_scatter_rows``   P -> S(0)                S(0) -> R
``all_reduce``            P -> R                   identity
``copy_to_tp``            identity                 P -> R (all-reduce)
========================  =======================  =========================
"""

from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["all_gather_rows", "reduce_scatter_rows", "all_reduce", "copy_to_tp", "all_gather_raw", "reduce_scatter_raw"]


def all_gather_raw(x: torch.Tensor, group, size: int) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty((x.shape[0] * size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_raw(x: torch.Tensor, group, size: int) -> torch.Tensor:
    x = x.contiguous()
    if x.shape[0] % size:
        raise ValueError(f"cannot scatter {x.shape[0]} rows over {size} ranks")
    out = torch.empty((x.shape[0] // size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return all_gather_raw(x, tp.group, tp.size)

    @staticmethod
    def backward(ctx, dy):
        return reduce_scatter_raw(dy, ctx.tp.group, ctx.tp.size), None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return reduce_scatter_raw(x, tp.group, tp.size)

    @staticmethod
    def backward(ctx, dy):
        return all_gather_raw(dy, ctx.tp.group, ctx.tp.size), None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=tp.group)
        return x

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous().clone()
        dist.all_reduce(dy, group=ctx.tp.group)
        return dy, None


def all_gather_rows(x, tp):
    return _AllGatherRows.apply(x, tp) if tp.size > 1 else x


def reduce_scatter_rows(x, tp):
    return _ReduceScatterRows.apply(x, tp) if tp.size > 1 else x


def all_reduce(x, tp):
    return _AllReduce.apply(x, tp) if tp.size > 1 else x


def copy_to_tp(x, tp):
    return _CopyToTP.apply(x, tp) if tp.size > 1 else x
