"""Context parallelism: tokens sharded over the cp group, K/V exchanged inside attention.

Sharding.  The ``T`` tokens of a microbatch are cut into ``2*cp`` chunks; with the
``headtail`` balancer rank r owns chunks ``r`` and ``2cp-1-r`` so causal work is even
(parity: torchtitan/distributed/context_parallel/api.py:137-226).  Inputs, labels and
positions are sharded identically; RoPE uses the (sharded) positions, the causal /
document mask uses the global token index ``q_pos`` of each local row.

Exchange modes
* ``allgather`` (the reference's scheme, decoder_sharding.py:263-302): K and V are
  all-gathered over cp (backward: reduce-scatter of dK, dV), re-ordered into sequence order,
  and each local query chunk attends to its causal prefix with a bottom-right aligned
  causal mask.
* ``ring``: K/V blocks travel around the cp ring (``batch_isend_irecv``) while each rank
  accumulates blockwise attention with the online-softmax (max / log-sum-exp) merge; only
  one remote block is resident at a time.  The output equals gathered-KV attention.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from torchtitan_b200.ops import functional as OF

from . import tp_ops

__all__ = ["CPContext", "shard_for_cp", "cp_attention", "cp_chunk_ids", "unshard_from_cp"]


@dataclass
class CPContext:
    group: object
    size: int
    rank: int
    mode: str = "allgather"  # allgather | ring
    load_balancer: str = "headtail"  # headtail | none
    nvlink: object | None = None  # parallel.cp_nvlink.CPNvlink: KV exchange by peer loads instead of NCCL


def cp_chunk_ids(cp: CPContext, rank: int | None = None) -> list[int]:
    r = cp.rank if rank is None else rank
    if cp.load_balancer == "headtail":
        return [r, 2 * cp.size - 1 - r]
    return [2 * r, 2 * r + 1]


def _local_index(cp: CPContext, T: int, device, rank: int | None = None) -> torch.Tensor:
    if T % (2 * cp.size):
        raise ValueError(f"token count {T} must be divisible by 2*cp = {2 * cp.size}")
    C = T // (2 * cp.size)
    return torch.cat([torch.arange(c * C, (c + 1) * C, device=device) for c in cp_chunk_ids(cp, rank)])


def shard_for_cp(cp: CPContext, tokens, positions, labels):
    """Returns the local slices and ``q_pos`` (global token index of each local row)."""
    idx = _local_index(cp, tokens.shape[-1], tokens.device)
    return tokens.index_select(-1, idx), positions.index_select(-1, idx), labels.index_select(-1, idx), idx


def unshard_from_cp(cp: CPContext, local: torch.Tensor) -> torch.Tensor:
    """All-gather rows over cp and restore sequence order (for tests / evaluation)."""
    full = tp_ops.all_gather_raw(local, cp.group, cp.size)
    T = full.shape[0]
    order = torch.cat([_local_index(cp, T, local.device, r) for r in range(cp.size)])
    out = torch.empty_like(full)
    out[order] = full
    return out


class _CPAllGather(torch.autograd.Function):
    """Gather rows over the cp group into *sequence order*; backward = reduce-scatter."""

    @staticmethod
    def forward(ctx, x, cp):
        ctx.cp = cp
        if cp.nvlink is not None and x.is_cuda:
            full = cp.nvlink.all_gather(x)
        else:
            full = tp_ops.all_gather_raw(x, cp.group, cp.size)
        T = full.shape[0]
        order = torch.cat([_local_index(cp, T, x.device, r) for r in range(cp.size)])
        ctx.order = order
        out = torch.empty_like(full)
        out[order] = full
        return out

    @staticmethod
    def backward(ctx, dy):
        cp = ctx.cp
        rank_major = dy.index_select(0, ctx.order).contiguous()
        if cp.nvlink is not None and dy.is_cuda:
            return cp.nvlink.reduce_scatter(rank_major), None
        return tp_ops.reduce_scatter_raw(rank_major, cp.group, cp.size), None


def _prefix_attention(q, k, v, n_prefix: int, scale: float):
    """One query chunk (the last ``Tq`` rows of the prefix) against ``k[:n_prefix]`` with a
    bottom-right aligned causal mask."""
    Tq = q.shape[0]
    kk, vv = k[:n_prefix], v[:n_prefix]
    if OF._native_attention_ok(q, kk, vv):
        # tcgen05 flash kernel: query row i sees keys j <= i + (n_prefix - Tq)
        from torchtitan_b200.ops.flash import flash_attention

        OF._count(4)
        return flash_attention(q, kk, vv, scale, causal=True, causal_offset=n_prefix - Tq)
    if q.is_cuda:
        from torch.nn.attention.bias import causal_lower_right

        qh, kh, vh = (t.transpose(0, 1).unsqueeze(0) for t in (q, kk, vv))
        out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=causal_lower_right(Tq, n_prefix), scale=scale,
                                             enable_gqa=(q.shape[1] != k.shape[1]))
        return out.squeeze(0).transpose(0, 1)
    q_pos = torch.arange(n_prefix - Tq, n_prefix, device=q.device)
    return OF._masked_attention(q, kk, vv, scale, True, None, None, None, q_pos, None)


def _block_attention_lse(q, k, v, scale, q_pos, k_pos, q_doc, k_doc, window):
    """Dense differentiable attention of a query block against one K/V block; returns the
    un-normalised pieces needed for the online-softmax merge: ``(out, lse)`` with
    ``lse = -inf`` for fully masked rows."""
    Hq, Hkv = q.shape[1], k.shape[1]
    rep = Hq // Hkv
    qh = q.transpose(0, 1).float()
    kh = k.transpose(0, 1).float()
    vh = v.transpose(0, 1).float()
    if rep > 1:
        kh, vh = kh.repeat_interleave(rep, 0), vh.repeat_interleave(rep, 0)
    s = torch.matmul(qh, kh.transpose(1, 2)) * scale
    mask = q_pos[:, None] >= k_pos[None, :]
    if window:
        mask &= (q_pos[:, None] - k_pos[None, :]) < window
    if q_doc is not None:
        mask &= q_doc[:, None] == k_doc[None, :]
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)  # [H, Tq]
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - safe[..., None])
    p = torch.where(mask[None], p, torch.zeros_like(p))
    return torch.matmul(p, vh), lse  # out [H, Tq, D]


def _merge(out_a, lse_a, out_b, lse_b):
    lse = torch.logaddexp(lse_a, lse_b)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    wa = torch.exp(lse_a - safe)[..., None]
    wb = torch.exp(lse_b - safe)[..., None]
    wa = torch.where(torch.isinf(lse_a)[..., None], torch.zeros_like(wa), wa)
    wb = torch.where(torch.isinf(lse_b)[..., None], torch.zeros_like(wb), wb)
    return out_a * wa + out_b * wb, lse


class _RingExchange(torch.autograd.Function):
    """Send ``x`` to the next rank of the ring and receive the previous rank's tensor."""

    @staticmethod
    def forward(ctx, x, cp):
        ctx.cp = cp
        return _ring_shift(x, cp, +1)

    @staticmethod
    def backward(ctx, dy):
        return _ring_shift(dy, ctx.cp, -1), None


def _ring_shift(x, cp: CPContext, direction: int):
    ranks = dist.get_process_group_ranks(cp.group)
    dst = ranks[(cp.rank + direction) % cp.size]
    src = ranks[(cp.rank - direction) % cp.size]
    x = x.contiguous()
    out = torch.empty_like(x)
    ops = [dist.P2POp(dist.isend, x, dst, group=cp.group), dist.P2POp(dist.irecv, out, src, group=cp.group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


def cp_attention(q, k, v, ctx, *, scale: float | None = None, window: int | None = None, sinks=None):
    """Attention of the local queries against the keys/values of the whole cp group."""
    cp: CPContext = ctx.cp
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if sinks is not None:
        raise NotImplementedError("attention sinks are not supported under context parallelism")
    Tl = q.shape[0]
    T = Tl * cp.size
    C = T // (2 * cp.size)
    q_pos = ctx.q_pos if ctx.q_pos is not None else _local_index(cp, T, q.device)
    plain = ctx.doc_ids is None and not window and cp.load_balancer == "headtail"

    if cp.mode == "allgather":
        kf = _CPAllGather.apply(k, cp)
        vf = _CPAllGather.apply(v, cp)
        if plain:
            outs = []
            for j, c in enumerate(cp_chunk_ids(cp)):
                outs.append(_prefix_attention(q[j * C:(j + 1) * C], kf, vf, (c + 1) * C, scale))
            return torch.cat(outs, dim=0)
        k_doc = None
        if ctx.doc_ids is not None:
            k_doc = unshard_from_cp(cp, ctx.doc_ids)
        k_pos = torch.arange(T, device=q.device)
        doc = None if k_doc is None else (ctx.doc_ids, k_doc)
        return OF._masked_attention(q, kf, vf, scale, True, doc, window, None, q_pos, k_pos)

    # ---- ring: blockwise accumulation while K/V circulate -------------------------------
    k_blk, v_blk = k, v
    pos_blk = q_pos
    doc_blk = ctx.doc_ids
    out = lse = None
    for step in range(cp.size):
        o, l = _block_attention_lse(q, k_blk, v_blk, scale, q_pos, pos_blk, ctx.doc_ids, doc_blk, window)
        out, lse = (o, l) if out is None else _merge(out, lse, o, l)
        if step + 1 < cp.size:
            k_blk = _RingExchange.apply(k_blk, cp)
            v_blk = _RingExchange.apply(v_blk, cp)
            with torch.no_grad():
                pos_blk = _ring_shift(pos_blk, cp, +1)
                if doc_blk is not None:
                    doc_blk = _ring_shift(doc_blk, cp, +1)
    return out.transpose(0, 1).to(q.dtype)
