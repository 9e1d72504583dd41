"""Expert-parallel token exchange over NVLink symmetric memory (``parallelism.ep_comm = "nvlink"``).

Instead of NCCL all-to-all + a local re-sort, every rank computes for each routing slot the rank
hosting the chosen expert and the row of that rank's receive buffer reserved for the slot (the
padded expert-major layout the grouped tcgen05 GEMMs consume), and

* dispatch: a kernel stores each token row straight into that row over NVLink (P2P stores);
* experts: grouped GEMMs run in place on the receive buffer;
* combine: a kernel pulls each token's K expert outputs from the peers (P2P loads), scales them
  by the gate values in fp32 and sums them: no atomics, no intermediate exchange buffers.

The backward mirrors it (scatter of ``w * dout``, local grouped backward, pull of ``dx``).  Only
the per-expert token counts travel through NCCL (an all-gather of ``E`` integers); one host read of
the local row total sizes the saved activations, as in the reference's all-to-all dispatcher
(torchtitan/models/common/token_dispatcher.py:245-370).  Each exchange is fenced by the bounded flag
barrier of the symmetric arena; buffer reuse across layers needs no extra barrier because a rank
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
    def __init__(self, group, device: torch.device, capacity_rows: int, dim: int):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.cap = (capacity_rows + 127) // 128 * 128
        self.dim = dim
        nbytes = 4 * (self.cap * dim * 2 + 512)
        self.arena = _GroupArena(group, device, nbytes)
        self.bufs = {}
        for name in ("x", "y", "dy", "dx"):
            t, off = self.arena.carve(self.cap * dim, torch.bfloat16)
            self.bufs[name] = (t.view(self.cap, dim), [b + off for b in self.arena.base_ptrs])

    def layout(self, selected: torch.Tensor, counts: torch.Tensor):
        """Destination (rank, row) of every routing slot and this rank's padded group offsets."""
        n, me = self.size, self.rank
        T, K = selected.shape
        E = counts.numel()
        El = E // n
        c = counts.to(torch.int64)
        all_c = torch.empty(n, E, dtype=torch.int64, device=c.device)
        dist.all_gather_into_tensor(all_c, c.contiguous(), group=self.group)
        tot = all_c.sum(0)
        padded = ((tot + (moe_ops.ALIGN - 1)) // moe_ops.ALIGN * moe_ops.ALIGN).view(n, El)
        offs = torch.zeros(n, El + 1, dtype=torch.int64, device=c.device)
        offs[:, 1:] = torch.cumsum(padded, dim=1)
        before_me = all_c[:me].sum(0)                                   # rows of lower ranks come first in a group
        base = offs[:, :-1].reshape(-1) + before_me                      # [E]: first row of my tokens for expert e
        flat = selected.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        e_sorted = flat[order]
        start = torch.cumsum(c, 0) - c
        pos = torch.arange(T * K, device=c.device) - start[e_sorted]
        dest_row = torch.empty(T * K, dtype=torch.int64, device=c.device)
        dest_row[order] = base[e_sorted] + pos
        dest_rank = flat // El
        my_offs = offs[me].to(torch.int32)
        my_counts = tot.view(n, El)[me].to(torch.int32)
        total = int(my_offs[-1])                                         # the one host read of this exchange
        if total > self.cap:
            raise RuntimeError(f"expert-parallel receive buffer overflow: {total} rows > capacity {self.cap}; raise "
                               "parallelism.ep_capacity_factor")
        return (dest_rank.view(T, K).to(torch.int32).contiguous(), dest_row.view(T, K).to(torch.int32).contiguous(),
                my_offs.contiguous(), my_counts.contiguous(), total)


class _EPNvlinkFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, top_scores, ep: EPNvlink, experts, dest_rank, dest_row, my_offs, my_counts, total):
        ops = ext.require()
        xbuf, xptrs = ep.bufs["x"]
        ybuf, yptrs = ep.bufs["y"]
        ops.ep_scatter_rows(x.contiguous(), dest_rank, dest_row, None, xptrs)
        ep.arena.barrier()
        ops.moe_zero_pad_rows(xbuf, my_offs, my_counts)
        with torch.enable_grad():
            x_loc = xbuf[:total].clone().requires_grad_(True)
            y_loc = experts.forward_padded(x_loc, my_offs)
        ybuf[:total].copy_(y_loc.detach())
        ep.arena.barrier()
        wts = top_scores.float().contiguous()
        out, keep = ops.ep_gather_rows(yptrs, dest_rank, dest_row, wts, x.shape[1], True, x)
        _count(4)
        ctx.save_for_backward(dest_rank, dest_row, my_offs, my_counts, wts, keep)
        ctx.local = (x_loc, y_loc)
        ctx.ep, ctx.total = ep, total
        return out

    @staticmethod
    def backward(ctx, dout):
        dest_rank, dest_row, my_offs, my_counts, wts, keep = ctx.saved_tensors
        x_loc, y_loc = ctx.local
        ep, total = ctx.ep, ctx.total
        ops = ext.require()
        dout = dout.contiguous()
        dw = ops.moe_slot_dot(dout, keep, wts.shape[1])
        dybuf, dyptrs = ep.bufs["dy"]
        dxbuf, dxptrs = ep.bufs["dx"]
        ops.ep_scatter_rows(dout, dest_rank, dest_row, wts, dyptrs)
        ep.arena.barrier()
        ops.moe_zero_pad_rows(dybuf, my_offs, my_counts)
        torch.autograd.backward(y_loc, dybuf[:total])
        dxbuf[:total].copy_(x_loc.grad)
        ep.arena.barrier()
        dx, _ = ops.ep_gather_rows(dxptrs, dest_rank, dest_row, None, dout.shape[1], False, dout)
        _count(4)
        ctx.local = None
        return dx, dw, None, None, None, None, None, None, None


def ep_experts_nvlink(ep: EPNvlink, experts, x: torch.Tensor, top_scores: torch.Tensor, selected: torch.Tensor,
                      counts: torch.Tensor) -> torch.Tensor:
    """Dispatch, grouped experts and weighted combine for tokens ``x[T, D]``; returns ``[T, D]``."""
    with torch.no_grad():
        dest_rank, dest_row, my_offs, my_counts, total = ep.layout(selected, counts)
    return _EPNvlinkFn.apply(x, top_scores, ep, experts, dest_rank, dest_row, my_offs, my_counts, total)
