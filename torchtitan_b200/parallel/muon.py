"""Distributed Muon on the flat-sharded engine.

Muon replaces the AdamW direction of a matrix parameter by the (approximate) polar factor of its
momentum, computed with a Newton-Schulz iteration: GEMM work on whole matrices, while the engine
stores every parameter as flat element ranges cut at arbitrary shard boundaries.  One step of a
unit therefore runs as

1. momentum update and Nesterov blend on this rank's flat shard (element-wise);
2. a packed all-to-all sends every piece of the blended bf16 shard to the owner of its matrix (split sizes
   from a static plan, no host read);
3. owner-computes: every matrix (a 2-D parameter, one ``block_rows`` x C row block of it, or one
   expert of a 3-D stack) has one owner rank, chosen by longest-processing-time-first balancing of
   the Newton-Schulz cost ``steps * short^2 * (2 long + short)``; the owner runs the iteration on
   the tensor-core GEMMs;
4. the reverse all-to-all brings each rank the directions of its own flat shard;
5. decoupled weight decay and the update, with the learning rate adjusted to the matrix shape,
   on the fp32 master shard; the compute-dtype copy is refreshed for the parameter all-gather.

Parity: torchtitan/distributed/flex_shard/dist_muon.py:252-640 (optimizer), :1810-1916 (the
learning-rate adjustment, momentum preparation, update and Newton-Schulz math).  The reference
moves matrices to their owners with a bucketed redistribution planner (:1889-1920); here the flat layout makes the
plan a list of contiguous pieces per (source, owner) pair.
"""

from __future__ import annotations

import heapq
import math
import re
from dataclasses import dataclass

import torch
import torch.distributed as dist

from torchtitan_b200.ops import functional as OF

__all__ = ["MUON_DEFAULTS", "newton_schulz", "adjust_lr", "muon_unit_step", "is_muon_group"]

MUON_DEFAULTS = dict(lr=1e-3, weight_decay=0.1, momentum=0.95, nesterov=True,
                     ns_coefficients=(3.4445, -4.7750, 2.0315), eps=1e-7, ns_steps=5, adjust_lr_fn=None,
                     block_rows={})


def is_muon_group(h: dict) -> bool:
    return h.get("optimizer_name") in ("DistMuon", "Muon")


def adjust_lr(lr: float, adjust_lr_fn: str | None, rows: int, cols: int) -> float:
    """Muon's learning rate for a ``rows x cols`` matrix."""
    if adjust_lr_fn is None or adjust_lr_fn == "original":
        ratio = math.sqrt(max(1.0, rows / cols))
    elif adjust_lr_fn == "match_rms_adamw":
        ratio = 0.2 * math.sqrt(max(rows, cols))
    elif adjust_lr_fn == "spectral_unclamped":
        ratio = math.sqrt(rows / cols)
    else:
        raise ValueError(f"unsupported adjust_lr_fn {adjust_lr_fn!r}")
    return lr * ratio


def newton_schulz(update: torch.Tensor, *, ns_coefficients=(3.4445, -4.7750, 2.0315), ns_steps: int = 5,
                  eps: float = 1e-7) -> torch.Tensor:
    """Approximate polar factor of a matrix (bf16 iteration, fp32 accumulation in the GEMMs).

    ``X <- a X + (b G + c G G) X`` with ``G = X X^T``, on the orientation whose Gram matrix is the
    smaller one, after scaling ``X`` to unit Frobenius norm."""
    a, b, c = ns_coefficients
    x = update.to(torch.bfloat16, copy=True)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t().contiguous()
    x = x / x.float().norm().clamp_min(eps).to(x.dtype)
    for _ in range(ns_steps):
        gram = OF.gemm_nt(x, x)                              # X X^T  [s, s]
        gu = (gram * b).contiguous()
        OF.gemm_nt(gram * c, gram, out=gu, accumulate=True)  # G symmetric: G G = G G^T
        xn = (x * a).contiguous()
        OF.gemm_nn(gu, x, out=xn, accumulate=True)
        x = xn
    return x.t() if transposed else x


@dataclass
class _Item:
    offset: int       # element offset of the matrix inside the unit's flat buffer
    rows: int
    cols: int
    group_idx: int
    owner: int = 0


def _plan_unit(u, groups: list[dict]) -> list[_Item]:
    """Matrices of the unit's Muon parameters with their owner ranks (identical on every rank)."""
    items: list[_Item] = []
    for s in u.slots:
        h = groups[s.group_idx]
        if not is_muon_group(h):
            continue
        if s.tp_slices is not None:
            raise ValueError(f"Muon on the tensor-parallel sharded parameter '{s.fqn}' is not supported: use tp = 1")
        shape = tuple(s.shape)
        if len(shape) == 2:
            block = 0
            for pat, rows in (h.get("block_rows") or {}).items():
                if re.search(pat, s.fqn):
                    block = int(rows)
                    break
            if block and shape[0] % block == 0 and block < shape[0]:
                for i in range(shape[0] // block):
                    items.append(_Item(s.offset + i * block * shape[1], block, shape[1], s.group_idx))
            else:
                items.append(_Item(s.offset, shape[0], shape[1], s.group_idx))
        elif len(shape) == 3:
            for e in range(shape[0]):
                items.append(_Item(s.offset + e * shape[1] * shape[2], shape[1], shape[2], s.group_idx))
        else:
            raise ValueError(f"Muon needs matrix parameters; '{s.fqn}' has shape {shape}")
    # longest processing time first onto the least loaded rank
    def cost(it: _Item) -> int:
        sd, ld = min(it.rows, it.cols), max(it.rows, it.cols)
        return int(groups[it.group_idx]["ns_steps"]) * sd * sd * (2 * ld + sd)

    heap = [(0, r) for r in range(u.size)]
    heapq.heapify(heap)
    for it in sorted(items, key=lambda t: (-cost(t), t.offset)):
        load, r = heapq.heappop(heap)
        it.owner = r
        heapq.heappush(heap, (load + cost(it), r))
    return items


def _a2a_plan(u, items):
    """Static exchange plan of a unit: which pieces of which rank's flat shard belong to matrices of which owner.

    ``send[o]``: ``(offset in my shard, length)`` pieces that go to owner ``o``; ``recv[s]``: ``(offset in my buffer of
    owned matrices, length)`` pieces that arrive from rank ``s``.  Both sides walk the matrices in flat order, so the
    pieces of a (source, owner) pair line up without any index exchange."""
    S = u.shard_numel
    owned_off, total = {}, 0
    for it in items:
        if it.owner == u.rank:
            owned_off[it.offset] = total
            total += it.rows * it.cols
    send = [[] for _ in range(u.size)]
    recv = [[] for _ in range(u.size)]
    for it in items:
        a0, b0 = it.offset, it.offset + it.rows * it.cols
        for s_ in range(a0 // S, min(u.size - 1, (b0 - 1) // S) + 1):
            a, b = max(a0, s_ * S), min(b0, (s_ + 1) * S)
            if a >= b:
                continue
            if s_ == u.rank:
                send[it.owner].append((a - s_ * S, b - a))
            if it.owner == u.rank:
                recv[s_].append((owned_off[it.offset] + (a - a0), b - a))
    return send, recv, owned_off, total


def _owner_compute_all_to_all(engine, u, items, groups, shard: torch.Tensor) -> torch.Tensor:
    """Matrices travel to their owners and the directions travel back with two packed all-to-alls: every element
    crosses the network once each way (an all-gather would deliver every matrix to every rank).  The split sizes come
    from the static plan, so nothing is read back to the host.  Parity: the packed all-to-all reshard of
    torchtitan/distributed/flex_shard/dist_muon.py:1889-1920."""
    plans = engine.__dict__.setdefault("_muon_a2a", {})
    if u.name not in plans:
        plans[u.name] = _a2a_plan(u, items)
    send, recv, owned_off, total = plans[u.name]
    dev = shard.device
    in_splits = [sum(n for _, n in send[o]) for o in range(u.size)]
    out_splits = [sum(n for _, n in recv[s_]) for s_ in range(u.size)]
    sendbuf = torch.empty(sum(in_splits), dtype=shard.dtype, device=dev)
    pos = 0
    for o in range(u.size):
        for off, n in send[o]:
            sendbuf[pos:pos + n].copy_(shard[off:off + n])
            pos += n
    recvbuf = torch.empty(sum(out_splits), dtype=shard.dtype, device=dev)
    dist.all_to_all_single(recvbuf, sendbuf, output_split_sizes=out_splits, input_split_sizes=in_splits, group=u.group)
    owned = torch.empty(total, dtype=shard.dtype, device=dev)
    pos = 0
    for s_ in range(u.size):
        for off, n in recv[s_]:
            owned[off:off + n].copy_(recvbuf[pos:pos + n])
            pos += n
    for it in items:
        if it.owner != u.rank:
            continue
        h = groups[it.group_idx]
        o0 = owned_off[it.offset]
        mat = owned[o0:o0 + it.rows * it.cols].view(it.rows, it.cols)
        mat.copy_(newton_schulz(mat, ns_coefficients=tuple(h["ns_coefficients"]), ns_steps=int(h["ns_steps"]),
                                eps=float(h["eps"])))
    # the way back: same pieces, roles swapped
    pos = 0
    for s_ in range(u.size):
        for off, n in recv[s_]:
            recvbuf[pos:pos + n].copy_(owned[off:off + n])
            pos += n
    dist.all_to_all_single(sendbuf, recvbuf, output_split_sizes=in_splits, input_split_sizes=out_splits, group=u.group)
    dshard = torch.zeros(u.shard_numel, dtype=shard.dtype, device=dev)
    pos = 0
    for o in range(u.size):
        for off, n in send[o]:
            dshard[off:off + n].copy_(sendbuf[pos:pos + n])
            pos += n
    return dshard


@torch.no_grad()
def muon_unit_step(engine, u, groups: list[dict], runs, step: int, grad_scale) -> None:
    """One optimizer step of a unit that holds Muon parameters (its AdamW runs included)."""
    from torchtitan_b200.ops import optim as optim_ops

    plans = engine.__dict__.setdefault("_muon_plans", {})
    if u.name not in plans:
        plans[u.name] = _plan_unit(u, groups)
    items: list[_Item] = plans[u.name]
    dev = u.master.device
    full = engine.__dict__.get("_muon_full")
    if full is None or full.numel() < u.padded:
        full = torch.empty(max(x.padded for x in engine.units), dtype=torch.bfloat16, device=dev)
        engine._muon_full = full
    full = full[:u.padded]
    shard = u.shard_view(full)
    shard.zero_()
    g = engine._grad_of(u)
    lowp = u.shard_view(u.flat_param)
    scale_t = grad_scale if isinstance(grad_scale, torch.Tensor) else None
    finite = torch.isfinite(scale_t).all() if scale_t is not None else None

    for gi, a, b in runs:
        h = groups[gi]
        if not is_muon_group(h):
            optim_ops.adamw_(u.master[a:b], g[a:b], u.exp_avg[a:b], u.exp_avg_sq[a:b], lowp[a:b],
                             lr=h["lr"], beta1=h["betas"][0], beta2=h["betas"][1], eps=h["eps"],
                             weight_decay=h["weight_decay"], step=step, grad_scale=grad_scale)
            continue
        gg = g[a:b].float() * (scale_t.reshape(()) if scale_t is not None else float(grad_scale))
        m = u.exp_avg[a:b]
        beta = float(h["momentum"])
        m_new = torch.lerp(m.float(), gg, 1.0 - beta)
        if finite is not None:   # a non-finite loss / gradient norm leaves the state untouched
            m_new = torch.where(finite, m_new, m.float())
        m.copy_(m_new)
        shard[a:b].copy_(torch.lerp(gg, m_new, beta) if h["nesterov"] else m_new)

    if u.size > 1:
        dshard = _owner_compute_all_to_all(engine, u, items, groups, shard)
    else:
        for it in items:
            h = groups[it.group_idx]
            mat = full[it.offset:it.offset + it.rows * it.cols].view(it.rows, it.cols)
            mat.copy_(newton_schulz(mat, ns_coefficients=tuple(h["ns_coefficients"]), ns_steps=int(h["ns_steps"]),
                                    eps=float(h["eps"])))
        dshard = full

    lo = u.shard_start
    for it in items:   # apply on the pieces of each matrix that fall into this rank's shard
        a, b = max(lo, it.offset), min(lo + u.shard_numel, it.offset + it.rows * it.cols)
        if a >= b:
            continue
        h = groups[it.group_idx]
        lr = float(h["lr"])
        seg = u.master[a - lo:b - lo]
        new = seg * (1.0 - lr * float(h["weight_decay"]))
        new.add_(dshard[a - lo:b - lo].float(), alpha=-adjust_lr(lr, h.get("adjust_lr_fn"), it.rows, it.cols))
        if finite is not None:
            new = torch.where(finite, new, seg)
        seg.copy_(new)
        lowp[a - lo:b - lo].copy_(seg)
