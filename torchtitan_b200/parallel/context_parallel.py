"""Context parallelism: tokens sharded over the cp group, K/V exchanged inside attention.

Sharding.  The ``T`` tokens of a microbatch are cut into ``2*cp`` chunks; with the
``headtail`` balancer rank r owns chunks ``r`` and ``2cp-1-r`` so causal work is even; the ``ptrr``
balancer cuts finer chunks and deals them by the work the batch's documents imply
(``ptrr_assignment``; parity: torchtitan/distributed/context_parallel/api.py:137-226).  Inputs, labels and
positions are sharded identically; RoPE uses the (sharded) positions, the causal /
document mask uses the global token index ``q_pos`` of each local row.

Exchange modes (both run every block on the flash-attention kernels, see ``_CPAttentionFn``)
* ``allgather`` (the reference's scheme, decoder_sharding.py:263-302): K and V are
  all-gathered over cp (backward: reduce-scatter of dK, dV), re-ordered into sequence order,
  and each local query chunk attends to its causal prefix with a bottom-right aligned
  causal mask (offset), the documents' first-key index and the sliding window.
* ``ring``: the K/V chunks of one rank at a time travel around the cp ring
  (``batch_isend_irecv``); every (query chunk, key chunk) block is attention with an offset,
  and the partial results are merged by their log-sum-exp (a small CUDA kernel); only one
  remote block is resident at a time.  The output equals gathered-KV attention.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from torchtitan_b200.ops import functional as OF

from . import tp_ops

__all__ = ["CPContext", "shard_for_cp", "cp_attention", "cp_chunk_ids", "unshard_from_cp", "ptrr_assignment"]


@dataclass
class CPContext:
    group: object
    size: int
    rank: int
    mode: str = "allgather"  # allgather | ring
    load_balancer: str = "headtail"  # headtail | ptrr | none
    nvlink: object | None = None  # parallel.cp_nvlink.CPNvlink: KV exchange by peer loads instead of NCCL
    assignment: list | None = None  # ptrr: chunk ids per rank for the current batch (``ptrr_assignment``)


def cp_chunk_ids(cp: CPContext, rank: int | None = None) -> list[int]:
    r = cp.rank if rank is None else rank
    if cp.assignment is not None:
        return list(cp.assignment[r])
    if cp.load_balancer in ("headtail", "ptrr"):
        return [r, 2 * cp.size - 1 - r]
    return [2 * r, 2 * r + 1]


def _num_chunks(cp: CPContext) -> int:
    return cp.size * len(cp_chunk_ids(cp, 0))


def _local_index(cp: CPContext, T: int, device, rank: int | None = None) -> torch.Tensor:
    n = _num_chunks(cp)
    if T % n:
        raise ValueError(f"token count {T} must be divisible by the number of context-parallel chunks ({n})")
    C = T // n
    return torch.cat([torch.arange(c * C, (c + 1) * C, device=device) for c in cp_chunk_ids(cp, rank)])


def ptrr_assignment(positions: torch.Tensor, cp_size: int, chunks_per_rank: int = 4) -> list[list[int]]:
    """Processing-time round-robin: cut the sequence into ``cp_size * chunks_per_rank`` chunks, estimate each chunk's
    attention work from the document structure (a token at position ``p`` of its document attends to ``p + 1``
    keys), sort the chunks by work and deal them to the ranks in snake order, heaviest first.  With packed documents
    of uneven length this balances better than the fixed head-tail pairing, which assumes one long causal sequence
    (parity: the reference's "ptrr" balancer, torchtitan/config/configs.py:246-255, built from the batch's mask).
    ``positions``: the batch's per-token positions ``[T]`` (host tensor); every rank computes the same answer."""
    T = positions.shape[-1]
    n = cp_size * chunks_per_rank
    if T % n:
        raise ValueError(f"token count {T} must be divisible by cp * chunks_per_rank = {n}")
    work = (positions.reshape(-1)[:T].to(torch.float64) + 1.0).view(n, T // n).sum(1)
    order = torch.argsort(work, descending=True, stable=True).tolist()
    out: list[list[int]] = [[] for _ in range(cp_size)]
    for i, c in enumerate(order):
        rnd, k = divmod(i, cp_size)
        out[k if rnd % 2 == 0 else cp_size - 1 - k].append(c)
    return [sorted(x) for x in out]


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


def _gather_sequence(x: torch.Tensor, cp: CPContext):
    """All ranks' rows in sequence order, and the index that maps rank-major rows to it."""
    if cp.nvlink is not None and x.is_cuda:
        full = cp.nvlink.all_gather(x)
    else:
        full = tp_ops.all_gather_raw(x, cp.group, cp.size)
    T = full.shape[0]
    order = torch.cat([_local_index(cp, T, x.device, r) for r in range(cp.size)])
    out = torch.empty_like(full)
    out[order] = full
    return out, order


def _scatter_sequence_grad(d_full: torch.Tensor, order: torch.Tensor, cp: CPContext, dtype) -> torch.Tensor:
    """Sum a sequence-ordered gradient over the cp group and keep this rank's rows."""
    rank_major = d_full.index_select(0, order).contiguous()
    if cp.nvlink is not None and rank_major.is_cuda:
        return cp.nvlink.reduce_scatter(rank_major.to(dtype)).to(dtype)
    return tp_ops.reduce_scatter_raw(rank_major, cp.group, cp.size).to(dtype)


def _apply_sinks(o32: torch.Tensor, lse: torch.Tensor, sinks: torch.Tensor):
    """A sink logit per head joins the denominator: ``lse' = logaddexp(lse, sink)``, ``o' = o exp(lse - lse')``."""
    lse2 = torch.logaddexp(lse, sinks.float()[:, None])
    w = torch.where(torch.isinf(lse), torch.zeros_like(lse), torch.exp(lse - lse2))
    return o32 * w.transpose(0, 1)[..., None], lse2


class _CPAttentionFn(torch.autograd.Function):
    """Context-parallel attention as a sum over (query chunk, key chunk) blocks.

    The local queries are ``2`` chunks of ``C`` consecutive tokens (global chunk ids ``cp_chunk_ids``); keys
    come in chunks of ``C`` consecutive tokens as well, so every block is plain causal attention with an offset:
    query ``i`` of chunk ``c`` sees key ``j`` of chunk ``c'`` iff ``j <= i + (c - c') C``.  Documents shift the
    per-row first visible key by ``c' C``; a sliding window keeps its meaning.  Blocks run on the flash kernels
    (``ops.flash.block_fwd``) and are merged by their log-sum-exp; the backward runs the flash backward of
    every block against the merged output and log-sum-exp, which is exact.

    ``allgather``: K/V are gathered into sequence order once and each query chunk attends to its prefix in one
    block (no merge).  ``ring``: the K/V chunks of one rank at a time travel around the ring together with their
    gradient accumulators."""

    @staticmethod
    def forward(ctx, q, k, v, sinks, cp, scale, window, kv_first, mode):
        from torchtitan_b200.ops import flash as FL

        Tl, Hq, D = q.shape
        ids = cp_chunk_ids(cp)
        C = Tl // len(ids)
        window = int(window or 0)
        o32 = torch.zeros(Tl, Hq, D, dtype=torch.float32, device=q.device)
        lse = torch.full((Hq, Tl), float("-inf"), dtype=torch.float32, device=q.device)
        saved_kv = None
        if mode == "allgather":
            kf, order = _gather_sequence(k, cp)
            vf, _ = _gather_sequence(v, cp)
            for j, c in enumerate(ids):
                n = (c + 1) * C
                o, l = FL.block_fwd(q[j * C:(j + 1) * C], kf[:n], vf[:n], scale, causal=True, causal_offset=c * C,
                                    kv_first=None if kv_first is None else kv_first[j * C:(j + 1) * C].contiguous(),
                                    window=window)
                o32[j * C:(j + 1) * C] = o.float()
                lse[:, j * C:(j + 1) * C] = l
            saved_kv = (kf, vf, order)
        else:
            for step, k_blk, v_blk in _ring_walk(cp, k, v):
                src_ids = cp_chunk_ids(cp, (cp.rank - step) % cp.size)
                _ring_blocks(FL.block_fwd, q, k_blk, v_blk, ids, src_ids, C, scale, window, kv_first,
                             lambda j, o, l: FL.merge_(o32[j * C:(j + 1) * C], lse[:, j * C:(j + 1) * C], o, l))
        if sinks is not None:
            o32, lse = _apply_sinks(o32, lse, sinks)
        o = o32.to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse, kv_first if kv_first is not None else torch.empty(0),
                              sinks if sinks is not None else torch.empty(0), *(saved_kv or ()))
        ctx.meta = (cp, scale, window, kv_first is not None, sinks is not None, mode)
        return o


    @staticmethod
    def backward(ctx, d_o):
        from torchtitan_b200.ops import flash as FL

        cp, scale, window, has_first, has_sinks, mode = ctx.meta
        q, k, v, o, lse, kv_first, sinks = ctx.saved_tensors[:7]
        kv_first = kv_first if has_first else None
        Tl, Hq, D = q.shape
        ids = cp_chunk_ids(cp)
        C = Tl // len(ids)
        d_o = d_o.contiguous()
        dq = torch.zeros(Tl, Hq, D, dtype=torch.float32, device=q.device)
        d_sinks = None
        if has_sinks:
            delta = (d_o.float() * o.float()).sum(-1)                                        # [Tl, Hq]
            d_sinks = -(torch.exp(sinks.float()[None, :] - lse.t()) * delta).sum(0).to(sinks.dtype)

        def chunk(t, j):
            return t[j * C:(j + 1) * C]

        if mode == "allgather":
            kf, vf, order = ctx.saved_tensors[7:10]
            dkf = torch.zeros(kf.shape, dtype=torch.float32, device=q.device)
            dvf = torch.zeros(vf.shape, dtype=torch.float32, device=q.device)
            for j, c in enumerate(ids):
                n = (c + 1) * C
                g = FL.block_bwd(chunk(d_o, j), chunk(q, j), kf[:n], vf[:n], chunk(o, j), lse[:, j * C:(j + 1) * C], scale,
                                 causal=True, causal_offset=c * C,
                                 kv_first=None if kv_first is None else chunk(kv_first, j).contiguous(), window=window)
                dq[j * C:(j + 1) * C] = g[0].float()
                dkf[:n] += g[1].float()
                dvf[:n] += g[2].float()
            dk = _scatter_sequence_grad(dkf, order, cp, k.dtype)
            dv = _scatter_sequence_grad(dvf, order, cp, v.dtype)
            return dq.to(q.dtype), dk, dv, d_sinks, None, None, None, None, None
        # ring: the K/V chunks come by again.  Over NCCL their gradient accumulators travel with them (one more hop
        # brings every accumulator home); over NVLink each rank keeps a full-size accumulator, indexed by source rank,
        # and one reduce-scatter by peer loads delivers every rank's rows.
        nv = cp.nvlink if (cp.nvlink is not None and k.is_cuda) else None
        n = cp.size
        if nv is not None:
            dk_all = torch.zeros((n,) + tuple(k.shape), dtype=torch.float32, device=q.device)
            dv_all = torch.zeros((n,) + tuple(v.shape), dtype=torch.float32, device=q.device)
        else:
            dk_acc = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
            dv_acc = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
        for step, k_blk, v_blk in _ring_walk(cp, k, v):
            src = (cp.rank - step) % n
            src_ids = cp_chunk_ids(cp, src)
            dk_t, dv_t = (dk_all[src], dv_all[src]) if nv is not None else (dk_acc, dv_acc)
            for j, c in enumerate(ids):
                for jj, c2 in enumerate(src_ids):
                    if c2 > c:
                        continue
                    kvf = None
                    if kv_first is not None:
                        kvf = (chunk(kv_first, j) - c2 * C).clamp_(min=0).to(torch.int32).contiguous()
                    g = FL.block_bwd(chunk(d_o, j), chunk(q, j), chunk(k_blk, jj), chunk(v_blk, jj), chunk(o, j),
                                     lse[:, j * C:(j + 1) * C], scale, causal=True, causal_offset=(c - c2) * C,
                                     kv_first=kvf, window=window)
                    dq[j * C:(j + 1) * C] += g[0].float()
                    dk_t[jj * C:(jj + 1) * C] += g[1].float()
                    dv_t[jj * C:(jj + 1) * C] += g[2].float()
            if nv is None:
                dk_acc, dv_acc = _ring_shift(dk_acc, cp, +1), _ring_shift(dv_acc, cp, +1)
        if nv is not None:
            dk_acc = nv.reduce_scatter(dk_all.view((n * k.shape[0],) + tuple(k.shape[1:])))
            dv_acc = nv.reduce_scatter(dv_all.view((n * v.shape[0],) + tuple(v.shape[1:])))
        return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), d_sinks, None, None, None, None, None


def _ring_walk(cp: CPContext, k: torch.Tensor, v: torch.Tensor):
    """Yields ``(step, k_block, v_block)``: at step ``s`` the K / V of rank ``rank - s``.

    NCCL: the blocks are passed around the ring with ``batch_isend_irecv``.  NVLink (``cp.nvlink``): every rank
    stages its K / V once in symmetric memory; the block of the next step is copied out of its owner's buffer on a
    side stream (a peer-to-peer copy, no SM involved) while the attention kernels work on the current block."""
    n = cp.size
    k_blk, v_blk = k.contiguous(), v.contiguous()
    nv = cp.nvlink if (cp.nvlink is not None and k.is_cuda) else None
    if nv is None:
        for step in range(n):
            yield step, k_blk, v_blk
            if step + 1 < n:
                k_blk, v_blk = _ring_shift(k_blk, cp, +1), _ring_shift(v_blk, cp, +1)
        return
    nv.stage_pair(k_blk, v_blk)
    main = torch.cuda.current_stream(k.device)
    side = getattr(nv, "_side_stream", None)
    if side is None:
        side = nv._side_stream = torch.cuda.Stream(k.device)
    nxt = None
    for step in range(n):
        if step + 1 < n:
            src = (cp.rank - step - 1) % n
            side.wait_stream(main)
            with torch.cuda.stream(side):
                pk, pv = nv.peer_pair(src, k_blk, v_blk)
                nk, nv_ = torch.empty_like(k_blk), torch.empty_like(v_blk)
                nk.copy_(pk)
                nv_.copy_(pv)
                ev = torch.cuda.Event()
                ev.record(side)
            nk.record_stream(main)
            nv_.record_stream(main)
            nxt = (nk, nv_, ev)
        yield step, k_blk, v_blk
        if step + 1 < n:
            main.wait_event(nxt[2])
            k_blk, v_blk = nxt[0], nxt[1]
    nv.release()


def _ring_blocks(block_fwd, q, k_blk, v_blk, ids, src_ids, C, scale, window, kv_first, sink):
    """Forward of every visible (local query chunk, held key chunk) block; ``sink(j, o, lse)`` merges it."""
    for j, c in enumerate(ids):
        for jj, c2 in enumerate(src_ids):
            if c2 > c:            # keys of a later chunk: nothing visible
                continue
            kvf = None
            if kv_first is not None:
                kvf = (kv_first[j * C:(j + 1) * C] - c2 * C).clamp_(min=0).to(torch.int32).contiguous()
            o, l = block_fwd(q[j * C:(j + 1) * C], k_blk[jj * C:(jj + 1) * C], v_blk[jj * C:(jj + 1) * C], scale,
                             causal=True, causal_offset=(c - c2) * C, kv_first=kvf, window=window)
            sink(j, o, l)


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


def _global_kv_first(cp: CPContext, ctx, T: int, device) -> torch.Tensor | None:
    """Global index of the first token of each local query's document (``None`` = one document)."""
    if getattr(ctx, "kv_first", None) is not None:
        return ctx.kv_first.to(torch.int32)
    if ctx.doc_ids is None:
        return None
    # document ids are non-decreasing along the sequence: the first position holding a query's id
    full = unshard_from_cp(cp, ctx.doc_ids.contiguous())
    return torch.searchsorted(full.contiguous(), ctx.doc_ids.contiguous(), right=False).to(torch.int32)


def cp_attention(q, k, v, ctx, *, scale: float | None = None, window: int | None = None, sinks=None):
    """Attention of the local queries against the keys/values of the whole cp group (causal; packed documents,
    sliding window and attention sinks supported in both exchange modes)."""
    cp: CPContext = ctx.cp
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    Tl = q.shape[0]
    if Tl % len(cp_chunk_ids(cp)):
        raise ValueError("the local token count must be a multiple of the number of chunks per rank")
    with torch.no_grad():
        kv_first = _global_kv_first(cp, ctx, Tl * cp.size, q.device)
    mode = "allgather" if cp.mode == "allgather" else "ring"
    return _CPAttentionFn.apply(q, k, v, sinks, cp, float(scale), window, kv_first, mode)
