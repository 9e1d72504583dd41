"""Muse Glimmer building blocks: gain-centred RMSNorm, attention with scale-free QK norm, a tuned
query scale, per-layer RoPE on/off (iRoPE), per-layer sliding window and a sigmoid output gate, and
a transformer block with pre- and post-norms around both sub-layers.
Parity: torchtitan/models/muse_glimmer/model.py:47-182.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from torchtitan_b200.models.common.attention import AttentionContext, GQAttention
from torchtitan_b200.models.common.decoder import TransformerBlock
from torchtitan_b200.models.common.layers import Linear, RMSNorm
from torchtitan_b200.models.common.module import InitSpec, Module, set_init
from torchtitan_b200.ops import functional as OF
from torchtitan_b200.parallel import tp_ops

__all__ = ["GainCenterRMSNorm", "MuseAttention", "MuseBlock", "EmbeddingNorm"]


class GainCenterRMSNorm(RMSNorm):
    """RMSNorm whose scale is ``weight + gain_center``; ``weight`` starts at zero."""

    @dataclass(kw_only=True, slots=True)
    class Config(RMSNorm.Config):
        gain_center: float = 1.0

    def __init__(self, config, **kw):
        super().__init__(config, **kw)
        set_init(self.weight, InitSpec(kind="zeros"))
        self.gain_center = config.gain_center

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return OF.rms_norm(x, self.weight + self.gain_center, self.eps)


class MuseAttention(GQAttention):
    @dataclass(kw_only=True, slots=True)
    class Config(GQAttention.Config):
        use_rope: bool = True
        scale_query_by: float = 1.0
        o_gate: Linear.Config | None = None

    def __init__(self, config, **kw):
        super().__init__(config, **kw)
        self.use_rope = config.use_rope
        self.scale_query_by = config.scale_query_by
        self.o_gate = None
        if config.o_gate is not None:
            config.o_gate.in_features, config.o_gate.out_features = config.dim, self.n_heads * self.head_dim
            self.o_gate = config.o_gate.build()

    def shard_(self, tp) -> None:
        super().shard_(tp)
        if self.o_gate is not None:
            self.o_gate.shard_("colwise", tp)

    def forward(self, x, positions, ctx: AttentionContext | None = None, norm: RMSNorm | None = None):
        tp = self.tp
        hd, hq, hkv = self.head_dim, self.n_heads, self.n_kv_heads
        if norm is not None:
            x = norm(x)
        if tp is not None:
            x = tp_ops.all_gather_rows(x, tp) if tp.sequence_parallel else tp_ops.copy_to_tp(x, tp)
        T = x.shape[0]
        qkv = self.wqkv(x).view(T, hq + 2 * hkv, hd)
        q = self.q_norm(qkv[:, :hq]) * self.scale_query_by
        k = self.k_norm(qkv[:, hq:hq + hkv])
        v = qkv[:, hq + hkv:]
        if self.use_rope:
            rp = ctx.rope_positions if ctx is not None and ctx.rope_positions is not None else positions
            q, k = self.rope(q, rp), self.rope(k, rp)
        ctx = ctx or AttentionContext()
        if ctx.kv_cache is not None:          # incremental decoding
            from torchtitan_b200.models.common.attention import cached_attention

            o = cached_attention(self, q, k, v, ctx.kv_cache, self.scale, window=int(self.window or 0))
        else:
            o = OF.attention(q, k, v, scale=self.scale, causal=True, doc_ids=ctx.doc_ids, window=self.window,
                             kv_first=ctx.kv_first)
        o = o.reshape(T, hq * hd)
        if self.o_gate is not None:
            o = o * torch.sigmoid(self.o_gate(x))
        y = self.wo(o)
        if tp is not None:
            return tp_ops.reduce_scatter_rows(y, tp) if tp.sequence_parallel else tp_ops.all_reduce(y, tp)
        return y


class MuseBlock(TransformerBlock):
    """``h = x + post_attn_norm(attn(attn_norm(x)));  out = h + post_ffn_norm(ffn(ffn_norm(h)))``."""

    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        post_attention_norm: RMSNorm.Config = field(default_factory=RMSNorm.Config)
        post_ffn_norm: RMSNorm.Config = field(default_factory=RMSNorm.Config)

    def __init__(self, config, **kw):
        super().__init__(config, **kw)
        self.post_attention_norm = config.post_attention_norm.build()
        self.post_ffn_norm = config.post_ffn_norm.build()

    def forward(self, x, positions, ctx=None):
        h = x + self.post_attention_norm(self.attention(x, positions, ctx, norm=self.attention_norm))
        return h + self.post_ffn_norm(self.feed_forward(self.ffn_norm(h)))


class EmbeddingNorm(Module):
    """Token embedding followed by a scale-free RMSNorm (kept together so that pipeline stages move both)."""

    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        num_embeddings: int = 0
        embedding_dim: int = 0
        init_std: float = 1.0
        eps: float = 1e-5

    def __init__(self, config, **_):
        super().__init__(config)
        from torchtitan_b200.models.common.layers import Embedding

        self.embedding = Embedding.Config(num_embeddings=config.num_embeddings, embedding_dim=config.embedding_dim,
                                          init_std=config.init_std).build()
        self.eps = config.eps

    @property
    def weight(self):
        return self.embedding.weight

    def shard_(self, tp) -> None:
        self.embedding.shard_(tp)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return OF.rms_norm(self.embedding(tokens), None, self.eps)
