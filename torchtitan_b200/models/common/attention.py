"""Grouped-query attention with a fused QKV projection.

The projection weight ``wqkv`` stacks ``[q heads | k heads | v heads]``; it is
saved to checkpoints as ``qkv_linear.wq/wk/wv`` (parity with the key layout of
torchtitan/models/common/attention.py:722-867).  RoPE is applied in place on the
packed projection output, q/k/v are strided views of it, and the pre-norm is
folded into the projection's autograd function.

Masking.  ``AttentionContext`` carries what the inner kernel needs: document ids
derived from ``positions`` (a document starts where ``positions == 0``), an
optional sliding window, and for context parallelism the global token indices of
this rank's queries.  (Reference: mask mods in attention.py:429-565, CP
placements in decoder_sharding.py:263-302.)
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from torchtitan_b200.ops import functional as OF
from torchtitan_b200.parallel import tp_ops

from .layers import Linear, RMSNorm, RoPE, TPContext
from .module import InitSpec, Module, set_init

__all__ = ["GQAttention", "AttentionContext", "KVCache", "BatchedKVCache", "cached_attention", "build_attention_context"]


@dataclass
class AttentionContext:
    doc_ids: torch.Tensor | None = None  # [T_local] int32, None = single document
    q_pos: torch.Tensor | None = None  # global token index of local rows (CP)
    cp: object | None = None  # parallel.context_parallel.CPContext
    max_doc_len: int | None = None
    kv_first: torch.Tensor | None = None  # [T_local] int32: index of the first token of each token's document
    rope_positions: torch.Tensor | None = None  # [3, T_local] multimodal rotary positions (overrides ``positions``)
    kv_cache: "KVCache | BatchedKVCache | None" = None  # incremental decoding: keys / values of earlier tokens, per attention layer


class KVCache:
    """Keys and values of the tokens seen so far, one pair of buffers per attention layer (incremental decoding
    with the training model itself; the reference's generator keeps its cache inside vLLM,
    torchtitan/experiments/rl).  Buffers grow in chunks; ``update`` appends the new rows and returns views of
    everything cached."""

    def __init__(self, chunk: int = 256):
        self.chunk = chunk
        self._k: dict[int, torch.Tensor] = {}
        self._v: dict[int, torch.Tensor] = {}
        self._len: dict[int, int] = {}

    def length(self, layer) -> int:
        return self._len.get(id(layer), 0)

    def state(self, layer) -> dict:
        """Free-form per-layer state for layers that are not attention (a recurrent layer's state matrix and the
        tail of its convolution inputs)."""
        if not hasattr(self, "_state"):
            self._state = {}
        return self._state.setdefault(id(layer), {})

    def update(self, layer, k: torch.Tensor, v: torch.Tensor):
        key = id(layer)
        n0, n = self._len.get(key, 0), k.shape[0]
        if key not in self._k or self._k[key].shape[0] < n0 + n:
            cap = (n0 + n + self.chunk - 1) // self.chunk * self.chunk
            nk = k.new_empty((cap,) + tuple(k.shape[1:]))
            nv = v.new_empty((cap,) + tuple(v.shape[1:]))
            if n0:
                nk[:n0], nv[:n0] = self._k[key][:n0], self._v[key][:n0]
            self._k[key], self._v[key] = nk, nv
        self._k[key][n0:n0 + n] = k
        self._v[key][n0:n0 + n] = v
        self._len[key] = n0 + n
        return self._k[key][:n0 + n], self._v[key][:n0 + n]


class BatchedKVCache:
    """Several sequences decoded in one forward pass: the flat token stream holds ``rows[i]`` consecutive rows of
    sequence ``i`` (its whole prompt at prefill, one row while decoding), each attending to its own ``caches[i]``.
    The projections and feed-forward layers run once over all rows; only the attention core is per sequence."""

    def __init__(self, caches: "list[KVCache]", rows: list[int]):
        assert len(caches) == len(rows)
        self.caches, self.rows = caches, rows


def cached_attention(layer, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_cache, scale: float, *, window: int = 0,
                     sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Append the new keys / values to ``layer``'s cache and attend the new queries to everything cached (causal
    among the new rows).  ``kv_cache``: one ``KVCache`` (all rows belong to one sequence) or a ``BatchedKVCache``
    (consecutive row blocks of several sequences).  Query / key and value head dimensions may differ (latent
    attention); shapes the flash kernels do not cover run the PyTorch block attention."""
    from torchtitan_b200.ops import flash as FL

    def attend(cache, q_, k_, v_):
        kc, vc = cache.update(layer, k_.detach(), v_.detach())
        o_, lse = FL.block_fwd(q_.contiguous(), kc, vc, scale, causal=True, causal_offset=kc.shape[0] - q_.shape[0],
                               window=window)
        if sinks is not None:
            o_ = (o_.float() * torch.sigmoid(lse - sinks.float()[:, None]).t()[..., None]).to(q_.dtype)
        return o_

    if not isinstance(kv_cache, BatchedKVCache):
        return attend(kv_cache, q, k, v)
    parts, r0 = [], 0
    for cache, n in zip(kv_cache.caches, kv_cache.rows):
        parts.append(attend(cache, q[r0:r0 + n], k[r0:r0 + n], v[r0:r0 + n]))
        r0 += n
    assert r0 == q.shape[0], f"BatchedKVCache rows cover {r0} of {q.shape[0]} tokens"
    return torch.cat(parts)


def build_attention_context(positions: torch.Tensor, *, assume_single_document: bool = False,
                            cp=None, q_pos: torch.Tensor | None = None) -> AttentionContext:
    """Derive document ids from ``positions`` (no host sync)."""
    if assume_single_document:
        return AttentionContext(None, q_pos, cp)
    starts = (positions == 0).to(torch.int32)
    doc_ids = torch.cumsum(starts, dim=0, dtype=torch.int32)
    # a document starts where positions == 0, so token i's document starts at (global index of i) - positions[i];
    # under context parallelism the rows are sharded and ``q_pos`` holds their global indices
    index = q_pos if (cp is not None and q_pos is not None) else torch.arange(positions.shape[0], device=positions.device)
    kv_first = (index - positions).to(torch.int32)
    return AttentionContext(doc_ids, q_pos, cp, kv_first=kv_first)


class GQAttention(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        n_heads: int = 0
        n_kv_heads: int | None = None
        head_dim: int | None = None
        wqkv: Linear.Config = field(default_factory=Linear.Config)
        wo: Linear.Config = field(default_factory=Linear.Config)
        qk_norm: RMSNorm.Config | None = None
        rope: RoPE.Config = field(default_factory=RoPE.Config)
        sliding_window: int | None = None
        use_sinks: bool = False
        softmax_scale: float | None = None

    def __init__(self, config: "GQAttention.Config", **_):
        super().__init__(config)
        c = config
        self.n_heads = c.n_heads
        self.n_kv_heads = c.n_kv_heads or c.n_heads
        self.head_dim = c.head_dim or c.dim // c.n_heads
        hd = self.head_dim
        c.wqkv.in_features = c.dim
        c.wqkv.out_features = (self.n_heads + 2 * self.n_kv_heads) * hd
        c.wqkv.row_blocks = [self.n_heads * hd, self.n_kv_heads * hd, self.n_kv_heads * hd]
        c.wo.in_features, c.wo.out_features = self.n_heads * hd, c.dim
        self.wqkv = c.wqkv.build()
        self.wo = c.wo.build()
        self.q_norm = self.k_norm = None
        if c.qk_norm is not None:
            c.qk_norm.dim = hd
            self.q_norm = c.qk_norm.build()
            self.k_norm = c.qk_norm.build()
        c.rope.dim = c.rope.dim or hd
        self.rope = c.rope.build()
        self.scale = c.softmax_scale if c.softmax_scale is not None else 1.0 / math.sqrt(hd)
        self.window = c.sliding_window
        self.sinks = None
        if c.use_sinks:
            self.sinks = nn.Parameter(torch.empty(self.n_heads))
            set_init(self.sinks, InitSpec(kind="trunc_normal", std=0.02))
        self.tp: TPContext | None = None

    # -- parallel ----------------------------------------------------------
    def shard_(self, tp: TPContext) -> None:
        if self.n_kv_heads % tp.size:
            raise ValueError(f"n_kv_heads={self.n_kv_heads} must divide by tp={tp.size}")
        self.wqkv.shard_("colwise", tp)
        self.wo.shard_("rowwise", tp)
        if self.sinks is not None:
            n = self.n_heads // tp.size
            s = nn.Parameter(torch.empty(n, device=self.sinks.device, dtype=self.sinks.dtype))
            s._tp_slices = (0, [(tp.rank * n, (tp.rank + 1) * n)], (self.n_heads,))
            set_init(s, self.sinks._init_spec)
            self.sinks = s
        self.n_heads //= tp.size
        self.n_kv_heads //= tp.size
        self.tp = tp

    def checkpoint_slices(self):
        hd = self.head_dim
        q, kv = self.n_heads * hd, self.n_kv_heads * hd
        out = {
            "wqkv.weight": [
                ("qkv_linear.wq.weight", 0, q),
                ("qkv_linear.wk.weight", q, q + kv),
                ("qkv_linear.wv.weight", q + kv, q + 2 * kv),
            ]
        }
        if self.wqkv.bias is not None:
            out["wqkv.bias"] = [
                ("qkv_linear.wq.bias", 0, q),
                ("qkv_linear.wk.bias", q, q + kv),
                ("qkv_linear.wv.bias", q + kv, q + 2 * kv),
            ]
        return out

    # -- forward -----------------------------------------------------------
    def forward(self, x: torch.Tensor, positions: torch.Tensor, ctx: AttentionContext | None = None,
                norm: RMSNorm | None = None) -> torch.Tensor:
        tp = self.tp
        hd, hq, hkv = self.head_dim, self.n_heads, self.n_kv_heads
        fused = False
        if tp is not None:
            if norm is not None:
                x = norm(x)
            fused = tp.fused_ok(x, self.wqkv, self.wo) and tp.fused.supported(x.shape[0] * tp.size, x.shape[1], hq * hd)
            if fused:
                from torchtitan_b200.parallel import tp_fused

                qkv = tp_fused.all_gather_linear(x, self.wqkv.weight, tp.fused)
            else:
                x = tp_ops.all_gather_rows(x, tp) if tp.sequence_parallel else tp_ops.copy_to_tp(x, tp)
                qkv = self.wqkv(x)
        elif type(norm) is RMSNorm and type(self.wqkv) is Linear and norm.weight is not None and self.wqkv.bias is None:
            qkv = OF.norm_linear(x, norm.weight, self.wqkv.weight, norm.eps)
        else:
            qkv = self.wqkv(norm(x) if norm is not None else x)
        T = qkv.shape[0]
        if ctx is not None and ctx.rope_positions is not None:
            positions = ctx.rope_positions          # multimodal: [3, T] temporal / height / width
        if self.q_norm is None:
            qkv = self.rope.apply_packed_(qkv, positions, hq + hkv, hd)
        qkv = qkv.view(T, hq + 2 * hkv, hd)
        if self.q_norm is not None:
            # QK-norm normalises each head vector before RoPE (Qwen3).
            qn = self.q_norm(qkv[:, :hq])
            kn = self.k_norm(qkv[:, hq:hq + hkv])
            q = self.rope(qn, positions)
            k = self.rope(kn, positions)
            v = qkv[:, hq + hkv:]
        else:
            q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
        ctx = ctx or AttentionContext()
        if ctx.kv_cache is not None:
            # incremental decoding (no autograd): the new queries attend to everything cached plus themselves
            o = cached_attention(self, q, k, v, ctx.kv_cache, self.scale, window=int(self.window or 0), sinks=self.sinks)
        elif ctx.cp is not None:
            from torchtitan_b200.parallel.context_parallel import cp_attention

            o = cp_attention(q, k, v, ctx, scale=self.scale, window=self.window, sinks=self.sinks)
        elif self.q_norm is None and self.window is None and self.sinks is None:
            o = OF.attention_packed(qkv, hq, hkv, self.scale, doc_ids=ctx.doc_ids, kv_first=ctx.kv_first)
        else:
            o = OF.attention(q, k, v, scale=self.scale, causal=True, doc_ids=ctx.doc_ids, window=self.window,
                             sinks=self.sinks, kv_first=ctx.kv_first)
        if fused:
            from torchtitan_b200.parallel import tp_fused

            return tp_fused.linear_reduce_scatter(o.reshape(T, hq * hd), self.wo.weight, tp.fused)
        y = self.wo(o.reshape(T, hq * hd))
        if tp is not None:
            return tp_ops.reduce_scatter_rows(y, tp) if tp.sequence_parallel else tp_ops.all_reduce(y, tp)
        return y
