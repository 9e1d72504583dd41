"""Expert-parallel token exchange over NVLink symmetric memory (``parallelism.ep_comm = "nvlink"``).

Instead of NCCL all-to-all + a local re-sort, every rank computes for each routing slot the rank
hosting the chosen expert and the row of that rank's receive buffer reserved for the slot (the
padded expert-major layout the grouped tcgen05 GEMMs consume), and

* dispatch: a kernel stores each token row straight into that row over NVLink (P2P stores);
* experts: grouped GEMMs run in place on the receive buffer;
* combine: a kernel pulls each token's K expert outputs from the peers (P2P loads), scales them
  by the gate values in fp32 and sums them: no atomics, no intermediate exchange buffers.

The backward mirrors it (scatter of ``w * dout``, local grouped backward, pull of ``dx``).  The
layout is computed on the device as well: every rank stores its per-expert token counts into a small
symmetric table of every peer, and after a flag barrier one kernel derives the destination rank and
row of every routing slot and this rank's group offsets (``ep_publish_counts`` / ``ep_layout``).  There
is no library collective and no sort anywhere in the exchange.  With ``parallelism.ep_capacity_factor > 0`` the
buffers have a static capacity (the factor times the balanced load) and nothing is read on the host, so a MoE layer
can be captured in a CUDA graph; a slot that does not fit is dropped and reported through the arena's status word
(bit 3), which the trainer polls (``parallelism.ep_overflow``).  With the default factor 0 the buffers hold the worst
case and each exchange reads the number of rows this rank received on the host (the exact mode: any routing
imbalance fits, e.g. a freshly initialised router; kept rows and expert activations have the received size).  (The reference's counterpart is its sync-free MinimalAsyncEP,
torchtitan/distributed/minimal_async_ep/api.py:174-385; its all-to-all dispatcher reads split sizes on
the host, torchtitan/models/common/token_dispatcher.py:245-370.)  Each exchange is fenced by the bounded
flag barrier of the symmetric arena; buffer reuse across layers needs no extra barrier because a rank
rewrites a peer's buffer only after a later barrier that the peer reaches after it finished reading.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from torchtitan_b200.ops import ext, moe_ops
from torchtitan_b200.ops.functional import _count

from .symm import _GroupArena

__all__ = ["EPNvlink", "ep_experts_nvlink"]


class EPNvlink:
    def __init__(self, group, device: torch.device, capacity_rows: int, dim: int, num_experts: int, exact: bool = False):
        """``exact``: the symmetric buffers hold the worst case (``capacity_rows`` = every routed row of every rank)
        and each exchange reads the number of rows this rank really received on the host, so that the rows kept
        for backward and the expert activations have that size: any routing imbalance fits, at the price of one
        host read per layer (no CUDA-graph capture).  Otherwise the capacity is static and nothing is read."""
        self.exact = exact
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.cap = (capacity_rows + 127) // 128 * 128
        self.dim = dim
        self.num_experts = num_experts
        nbytes = 4 * (self.cap * dim * 2 + 512) + 4 * self.size * num_experts + 512
        self.arena = _GroupArena(group, device, nbytes)
        # counts[src rank][expert], written by the peers
        self.table, off = self.arena.carve(self.size * num_experts, torch.int32)
        self.table = self.table.view(self.size, num_experts)
        self.table.zero_()
        self.table_ptrs = [b + off for b in self.arena.base_ptrs]
        self.bufs = {}
        for name in ("x", "y", "dy", "dx"):
            t, off = self.arena.carve(self.cap * dim, torch.bfloat16)
            self.bufs[name] = (t.view(self.cap, dim), [b + off for b in self.arena.base_ptrs])

    def layout(self, selected: torch.Tensor, counts: torch.Tensor):
        """Destination (rank, row) of every routing slot and this rank's padded group offsets, on the device."""
        ops = ext.require()
        if counts.numel() != self.num_experts:
            raise ValueError(f"expected counts of {self.num_experts} experts, got {counts.numel()}")
        ops.ep_publish_counts(counts.float().contiguous(), self.table_ptrs, self.rank)
        self.arena.barrier()                       # every rank's row of the table has landed
        _count(2)
        dest_rank, dest_row, my_offs, my_counts = ops.ep_layout(selected.to(torch.int32).contiguous(), self.table, self.rank,
                                                                self.cap, moe_ops.ALIGN, self.arena.status)
        return dest_rank, dest_row, my_offs, my_counts


def _plain_experts(experts) -> bool:
    """Plain bf16 grouped SwiGLU experts: the exchange calls their forward / backward directly, with the symmetric
    buffers as the GEMM outputs.  Anything else (quantised recipes, other expert classes) runs as a nested autograd
    graph on copies."""
    return (type(experts).__name__ == "GroupedExperts" and not getattr(experts, "quant_recipe", None)
            and all(hasattr(experts, n) for n in ("w1_EFD", "w3_EFD", "w2_EDF")))


class _EPNvlinkFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, top_scores, ep: EPNvlink, experts, dest_rank, dest_row, my_offs, my_counts, *weights):
        ops = ext.require()
        xbuf, xptrs = ep.bufs["x"]
        ybuf, yptrs = ep.bufs["y"]
        ops.ep_scatter_rows(x.contiguous(), dest_rank, dest_row, None, xptrs)
        ep.arena.barrier()
        R = ep.cap
        if ep.exact:
            # rows this rank received, padded per expert (the one host read of the exact mode)
            R = max(moe_ops.ALIGN, min(ep.cap, int(my_offs[-1])))
            xbuf, ybuf = xbuf[:R], ybuf[:R]
        ctx.rows = R
        ops.moe_zero_pad_rows(xbuf, my_offs, my_counts)
        # the whole static buffer is kept for the weight gradients (the next layer's dispatch overwrites xbuf): rows
        # at or beyond my_offs[-1] are never read by the grouped GEMMs
        ctx.plain = bool(weights)
        if ctx.plain:
            w1, w3, w2 = weights
            x_loc = xbuf.clone()
            _, gu = moe_ops.swiglu_experts_fwd(x_loc, w1, w3, w2, my_offs, out=ybuf)   # the last GEMM writes ybuf
            ctx.local = (x_loc, gu)
            ctx.weights = weights
        else:
            with torch.enable_grad():
                x_loc = xbuf.clone().requires_grad_(True)
                y_loc = experts.forward_padded(x_loc, my_offs)
            ybuf.copy_(y_loc.detach())
            ctx.local = (x_loc, y_loc)
        ep.arena.barrier()
        wts = top_scores.float().contiguous()
        out, keep = ops.ep_gather_rows(yptrs, dest_rank, dest_row, wts, x.shape[1], True, x)
        _count(4)
        ctx.save_for_backward(dest_rank, dest_row, my_offs, my_counts, wts, keep)
        ctx.ep = ep
        return out

    @staticmethod
    def backward(ctx, dout):
        dest_rank, dest_row, my_offs, my_counts, wts, keep = ctx.saved_tensors
        ep = ctx.ep
        ops = ext.require()
        dout = dout.contiguous()
        dw = ops.moe_slot_dot(dout, keep, wts.shape[1])
        dybuf, dyptrs = ep.bufs["dy"]
        dxbuf, dxptrs = ep.bufs["dx"]
        ops.ep_scatter_rows(dout, dest_rank, dest_row, wts, dyptrs)
        ep.arena.barrier()
        dybuf, dxbuf = dybuf[:ctx.rows], dxbuf[:ctx.rows]
        ops.moe_zero_pad_rows(dybuf, my_offs, my_counts)
        wgrads = ()
        if ctx.plain:
            x_loc, gu = ctx.local
            w1, w3, w2 = ctx.weights
            # the input-gradient GEMMs write dxbuf; weight gradients go to main_grad (or come back for autograd)
            _, dw1, dw3, dw2 = moe_ops.swiglu_experts_bwd(dybuf, x_loc, gu, w1, w3, w2, my_offs, need_dx=True, dx_out=dxbuf)
            wgrads = (dw1, dw3, dw2)
            ctx.weights = None
        else:
            x_loc, y_loc = ctx.local
            torch.autograd.backward(y_loc, dybuf)
            dxbuf.copy_(x_loc.grad)
        ep.arena.barrier()
        dx, _ = ops.ep_gather_rows(dxptrs, dest_rank, dest_row, None, dout.shape[1], False, dout)
        _count(4)
        ctx.local = None
        return (dx, dw, None, None, None, None, None, None) + wgrads


def ep_experts_nvlink(ep: EPNvlink, experts, x: torch.Tensor, top_scores: torch.Tensor, selected: torch.Tensor,
                      counts: torch.Tensor) -> torch.Tensor:
    """Dispatch, grouped experts and weighted combine for tokens ``x[T, D]``; returns ``[T, D]``."""
    with torch.no_grad():
        dest_rank, dest_row, my_offs, my_counts = ep.layout(selected, counts)
    weights = (experts.w1_EFD, experts.w3_EFD, experts.w2_EDF) if _plain_experts(experts) else ()
    return _EPNvlinkFn.apply(x, top_scores, ep, experts, dest_rank, dest_row, my_offs, my_counts, *weights)
