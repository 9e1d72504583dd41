"""Expert parallelism: all-to-all token dispatch / combine around the local grouped experts.

Baseline exchange (``ep_comm="nccl"``), the standard token-choice protocol of the reference
(torchtitan/models/common/token_dispatcher.py:245-370,501-559):

1. rows arrive sorted by *global* expert id, i.e. rank-major for the ep group;
2. per-expert counts are exchanged with an all-to-all, the host reads the split sizes;
3. rows travel with a variable-split all-to-all; the receiver re-sorts them from
   (source rank, local expert) to local-expert-major and builds the grouped-GEMM offsets;
4. expert outputs take the inverse permutation and the inverse all-to-all.

Both exchanges are autograd functions whose backward is the opposite exchange.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

__all__ = ["EPContext", "apply_expert_parallel", "ep_experts"]


@dataclass
class EPContext:
    group: object
    size: int
    rank: int
    comm: str = "nccl"
    nvlink: object | None = None  # parallel.ep_nvlink.EPNvlink when comm == "nvlink" on CUDA


def apply_expert_parallel(model, pdims, parallelism) -> None:
    ep = EPContext(group=pdims.group("ep"), size=pdims.ep, rank=pdims.local_rank("ep"), comm=parallelism.ep_comm)
    if ep.comm == "nvlink" and torch.cuda.is_available():
        from .symm import symm_available

        if symm_available():
            from .ep_nvlink import EPNvlink

            moes = [blk.moe for blk in model.layers.values() if blk.moe is not None]
            if moes:
                t = getattr(parallelism, "_tokens_per_rank", 0) or 8192
                k, e_local = moes[0].config.top_k, moes[0].num_experts // ep.size
                # rows a rank can receive: capacity factor x the balanced load plus the alignment padding of its
                # experts.  Factor 0 (the default): buffers for the worst case (every token of every rank) and the
                # received row count read on the host per exchange, so that any imbalance fits
                exact = not parallelism.ep_capacity_factor
                factor = parallelism.ep_capacity_factor or float(ep.size)
                cap = int(factor * t * k) + e_local * 128
                ep.nvlink = EPNvlink(ep.group, torch.device("cuda", torch.cuda.current_device()), cap, moes[0].config.dim,
                                     moes[0].num_experts, exact=exact)
    for blk in model.layers.values():
        if blk.moe is not None:
            blk.moe.routed_experts.ep = ep
            blk.moe.routed_experts.inner_experts.shard_experts_(ep.size, ep.rank)


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all of rows; the backward swaps the split lists."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = dy.new_empty((sum(ctx.in_splits), *dy.shape[1:]))
        dist.all_to_all_single(dx, dy.contiguous(), output_split_sizes=ctx.in_splits,
                               input_split_sizes=ctx.out_splits, group=ctx.group)
        return dx, None, None, None


def ep_experts(ep: EPContext, experts, rows: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """``rows[N, D]`` sorted by global expert id, ``counts[E]`` (fp32 histogram of this rank's
    routing).  Returns the expert outputs in the same row order."""
    E_local = experts.num_experts
    n = ep.size
    with torch.no_grad():
        send_counts = counts.to(torch.int64).view(n, E_local)  # [dst rank, local expert]
        recv_counts = torch.empty_like(send_counts)  # [src rank, local expert]
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=ep.group)
        # the split sizes must be known on the host (the one sync of this protocol)
        both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
        in_splits, out_splits = both[0].tolist(), both[1].tolist()
    recv = _AllToAllRows.apply(rows, in_splits, out_splits, ep.group)
    with torch.no_grad():
        # received rows are ordered (src rank, local expert); reorder to local-expert-major
        seg = recv_counts.reshape(-1)  # length n * E_local, segment s = src * E_local + e
        seg_expert = torch.arange(n * E_local, device=rows.device) % E_local
        row_expert = torch.repeat_interleave(seg_expert, seg, output_size=recv.shape[0])
    if experts.native_ok(recv):
        # padded expert-major layout for the tcgen05 grouped GEMMs (own permute / gather kernels)
        from torchtitan_b200.ops import moe_ops

        with torch.no_grad():
            dest, offs_pad, cap = moe_ops.padded_layout(row_expert.view(-1, 1), recv_counts.sum(0).float())
        xp = moe_ops.permute_rows(recv, dest, cap)
        yp = experts.forward_padded(xp, offs_pad)
        back = moe_ops.gather_rows(yp, dest)
        return _AllToAllRows.apply(back, out_splits, in_splits, ep.group)
    with torch.no_grad():
        perm = torch.argsort(row_expert, stable=True)
        offs = torch.cumsum(recv_counts.sum(0), 0).to(torch.int32)
    x = recv.index_select(0, perm)
    y = experts(x, offs)
    back = torch.empty_like(y)
    back = back.index_copy(0, perm, y)
    return _AllToAllRows.apply(back, out_splits, in_splits, ep.group)
