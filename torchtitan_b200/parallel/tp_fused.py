"""Tensor-parallel linears whose collective runs inside the GEMM kernel (async tensor parallelism).

``all_gather_linear``: sequence-sharded activations ``x[T/R, K]`` times a column-parallel weight.
Every rank writes its rows into its slot of a symmetric gather buffer; after one flag barrier the
GEMM kernel starts on the local rows while 128 extra threads per CTA pull the other ranks' rows over
NVLink in 128-row blocks, and row tiles wait for the flag of their block.  ``linear_reduce_scatter``:
a row-parallel weight; the GEMM epilogue stores every output tile into the staging buffer of the
rank that owns those rows (TMA stores to peer memory), and after a barrier a small kernel sums the
``R`` staged slots.  The backward of each is the other (plus a local weight-gradient GEMM).

The reference reaches the same overlap with ``torch.ops.symm_mem.fused_all_gather_matmul`` /
``fused_matmul_reduce_scatter`` (torchtitan/distributed/linear.py:47-421); here the collective and
the tcgen05 tiles are one kernel.  Buffers are double buffered per shape, so one barrier per call
is enough: a slot is rewritten two calls later, after every rank has passed the barrier in between.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from torchtitan_b200.ops import ext, functional as OF
from torchtitan_b200.ops.functional import _count

from .symm import _GroupArena

__all__ = ["FusedTP", "all_gather_linear", "linear_reduce_scatter"]


class FusedTP:
    """Symmetric buffers of one tensor-parallel group."""

    def __init__(self, group, device: torch.device, nbytes: int = 1 << 30):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.arena = _GroupArena(group, device, nbytes)
        self._bufs: dict[tuple, list] = {}
        self._turn: dict[tuple, int] = {}
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)   # device counter, advanced with each gather barrier

    def supported(self, rows: int, *dims: int) -> bool:
        return rows % (256 * self.size) == 0 and all(d % 8 == 0 for d in dims)

    def _pair(self, kind: str, rows: int, cols: int):
        """Two symmetric ``[rows, cols]`` bf16 buffers (with peer pointers and flags), used alternately."""
        key = (kind, rows, cols)
        if key not in self._bufs:
            pair = []
            for _ in range(2):
                t, off = self.arena.carve(rows * cols, torch.bfloat16)
                ptrs = [b + off for b in self.arena.base_ptrs]
                flags = torch.zeros(max(1, rows // 128), dtype=torch.int32, device=self.device)
                pair.append((t.view(rows, cols), ptrs, flags))
            self._bufs[key] = pair
            self._turn[key] = 0
        i = self._turn[key]
        self._turn[key] = i ^ 1
        return self._bufs[key][i]

    # -- raw operations (no autograd) ------------------------------------------------------
    def ag_gemm(self, x_shard: torch.Tensor, b: torch.Tensor, mode: int):
        """Returns ``(gathered . b, gathered)``; ``gathered`` is the symmetric buffer (valid until reused)."""
        S, K = x_shard.shape
        T = S * self.size
        buf, ptrs, flags = self._pair("gather", T, K)
        buf[self.rank * S:(self.rank + 1) * S].copy_(x_shard)
        self.arena.barrier(bump=self.epoch)
        N = b.shape[0] if mode == 0 else b.shape[1]
        out = torch.empty(T, N, dtype=x_shard.dtype, device=x_shard.device)
        _count()
        ext.require().gemm_allgather_bf16(buf, b, out, ptrs, self.rank, flags, self.epoch, mode)
        return out, buf

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, mode: int) -> torch.Tensor:
        T = a.shape[0]
        N = b.shape[0] if mode == 0 else b.shape[1]
        staging, ptrs, _ = self._pair("staging", T, N)   # [R, T/R, N] viewed as [T, N]
        _count(2)
        ops = ext.require()
        ops.gemm_scatter_bf16(a, b, ptrs, self.rank, mode)
        self.arena.barrier()
        return ops.sum_slots(staging.view(self.size, T // self.size, N))


class _AllGatherLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, ftp):
        y, gathered = ftp.ag_gemm(x_shard.contiguous(), weight, 0)
        ctx.save_for_backward(gathered.clone(), weight)   # the buffer itself is reused by later layers
        ctx.ftp = ftp
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = ctx.ftp.gemm_rs(dy, weight, 1) if ctx.needs_input_grad[0] else None   # dy . W, rows scattered
        dw = OF._wgrad(dy, x_full, weight) if weight.requires_grad else None
        return dx, dw, None


class _LinearReduceScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, ftp):
        x = x.contiguous()
        y = ftp.gemm_rs(x, weight, 0)
        ctx.save_for_backward(x, weight)
        ctx.ftp = ftp
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        dx, dy_full = ctx.ftp.ag_gemm(dy_shard.contiguous(), weight, 1)   # gathered dy . W
        dw = OF._wgrad(dy_full, x, weight) if weight.requires_grad else None
        return (dx if ctx.needs_input_grad[0] else None), dw, None


def all_gather_linear(x_shard: torch.Tensor, weight: torch.Tensor, ftp: FusedTP) -> torch.Tensor:
    """``all_gather(x_shard) @ weight^T`` with ``x_shard[T/R, K]`` and ``weight[N_local, K]``."""
    return _AllGatherLinearFn.apply(x_shard, weight, ftp)


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, ftp: FusedTP) -> torch.Tensor:
    """``reduce_scatter(x @ weight^T)`` over rows with ``x[T, K_local]`` and ``weight[N, K_local]``."""
    return _LinearReduceScatterFn.apply(x, weight, ftp)
