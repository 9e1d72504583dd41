"""Multi-head latent attention (DeepSeek-V2/V3, Kimi).

Queries optionally go through a low-rank bottleneck (``wq_a -> q_norm -> wq_b``); keys and
values are expanded per head from a shared compressed latent (``wkv_a -> kv_norm -> wkv_b``)
plus one rotary key head shared by all query heads.  The rotary part uses the interleaved
("complex") convention with YaRN scaling; when the rope factor is > 1 the softmax scale is
multiplied by ``mscale^2`` with ``mscale = 0.1 * mscale_cfg * ln(factor) + 1``.
Parity: torchtitan/models/deepseek_v3/model.py:28-233 (parameter names ``wq_a, q_norm, wq_b,
wq, wkv_a, kv_norm, wkv_b, wo``).

The query/key head dimension (nope + rope, 192 for the released models) differs from the value
head dimension (128), so the inner attention pads values up to the query width and runs the
tcgen05 kernel when that width is 128, and the general masked path otherwise.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from torchtitan_b200.ops import functional as OF
from torchtitan_b200.parallel import tp_ops

from .attention import AttentionContext
from .layers import Linear, RMSNorm, RoPE, TPContext
from .module import Module

__all__ = ["MLAttention"]


class _MLAAssembleFn(torch.autograd.Function):
    """Rotary embedding of the decoupled query / key parts and assembly of ``qf``, ``kf``, ``v`` in one kernel
    (``ops/csrc/mla.cu``); the backward is its transpose (the gradient of the shared rotary key sums over the heads)."""

    @staticmethod
    def forward(ctx, q, kv, k_pe, table, positions, dn, dr, dv):
        from torchtitan_b200.ops import ext
        from torchtitan_b200.ops.functional import _count

        pos = positions.to(torch.int64).contiguous()
        ctx.save_for_backward(table, pos)
        ctx.dims = (dn, dr, dv)
        _count()
        return ext.require().mla_assemble_fwd(q.contiguous(), kv.contiguous(), k_pe, table, pos, dn, dr, dv)

    @staticmethod
    def backward(ctx, dqf, dkf, dv_):
        from torchtitan_b200.ops import ext
        from torchtitan_b200.ops.functional import _count

        table, pos = ctx.saved_tensors
        dn, dr, dv = ctx.dims
        _count()
        dq, dkv, dk_pe = ext.require().mla_assemble_bwd(dqf.contiguous(), dkf.contiguous(), dv_.contiguous(), table, pos,
                                                        dn, dr, dv)
        return dq, dkv, dk_pe, None, None, None, None, None


def _assemble_kernel_ok(q, kv, kv_a, positions, rope, dn, dr, dv, rank) -> bool:
    from torchtitan_b200.ops import ext

    return (q.is_cuda and q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and positions.dim() == 1
            and rope.interleaved and rope.cache.shape[1] == dr and rope.cache.dtype == torch.float32
            and dn % 8 == 0 and dr % 8 == 0 and dv % 8 == 0 and rank % 8 == 0 and kv_a.shape[1] % 8 == 0
            and ext.available())


class MLAttention(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        n_heads: int = 0
        q_lora_rank: int = 0
        kv_lora_rank: int = 512
        qk_nope_head_dim: int = 128
        qk_rope_head_dim: int = 64
        v_head_dim: int = 128
        norm_eps: float = 1e-6
        mscale: float = 1.0
        init_std: float = 0.02
        out_init_std: float = 0.02
        rope: RoPE.Config = field(default_factory=RoPE.Config)
        # present for interface parity with GQAttention.Config
        n_kv_heads: int | None = None
        head_dim: int | None = None
        qk_norm: object | None = None
        use_sinks: bool = False
        wqkv: Linear.Config = field(default_factory=Linear.Config)
        wo: Linear.Config = field(default_factory=Linear.Config)

    def __init__(self, config: "MLAttention.Config", **_):
        super().__init__(config)
        c = config
        self.n_heads = c.n_heads
        self.qk_head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        L = Linear.Config
        if c.q_lora_rank:
            self.wq_a = L(in_features=c.dim, out_features=c.q_lora_rank, init_std=c.init_std).build()
            self.q_norm = RMSNorm.Config(dim=c.q_lora_rank, eps=c.norm_eps).build()
            self.wq_b = L(in_features=c.q_lora_rank, out_features=c.n_heads * self.qk_head_dim, init_std=c.init_std).build()
            self.wq = None
        else:
            self.wq = L(in_features=c.dim, out_features=c.n_heads * self.qk_head_dim, init_std=c.init_std).build()
            self.wq_a = self.q_norm = self.wq_b = None
        self.wkv_a = L(in_features=c.dim, out_features=c.kv_lora_rank + c.qk_rope_head_dim, init_std=c.init_std).build()
        self.kv_norm = RMSNorm.Config(dim=c.kv_lora_rank, eps=c.norm_eps).build()
        self.wkv_b = L(in_features=c.kv_lora_rank, out_features=c.n_heads * (c.qk_nope_head_dim + c.v_head_dim),
                       init_std=c.init_std).build()
        self.wo = L(in_features=c.n_heads * c.v_head_dim, out_features=c.dim, init_std=c.out_init_std).build()
        c.rope.dim = c.qk_rope_head_dim
        self.rope = c.rope.build()
        self.scale = self.qk_head_dim ** -0.5
        if c.rope.scaling == "yarn" and c.rope.rope_factor > 1.0:
            m = 0.1 * c.mscale * math.log(c.rope.rope_factor) + 1.0
            self.scale *= m * m
        self.tp: TPContext | None = None
        # the low-rank projections see every token and are small: replicated under tensor parallelism
        for mod in (self.wq_a, self.q_norm, self.wkv_a, self.kv_norm):
            if mod is not None:
                for p in mod.parameters():
                    p._replicated_over_tp = True

    def shard_(self, tp: TPContext) -> None:
        if self.n_heads % tp.size:
            raise ValueError(f"n_heads={self.n_heads} must divide by tp={tp.size}")
        (self.wq_b if self.wq_b is not None else self.wq).shard_("colwise", tp)
        self.wkv_b.shard_("colwise", tp)
        self.wo.shard_("rowwise", tp)
        self.n_heads //= tp.size
        self.tp = tp

    def forward(self, x: torch.Tensor, positions: torch.Tensor, ctx: AttentionContext | None = None,
                norm: RMSNorm | None = None) -> torch.Tensor:
        c = self.config
        tp = self.tp
        if norm is not None:
            x = norm(x)
        if tp is not None:
            x = tp_ops.all_gather_rows(x, tp) if tp.sequence_parallel else tp_ops.copy_to_tp(x, tp)
        T = x.shape[0]
        H, dn, dr, dv = self.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
        q = self.wq_b(self.q_norm(self.wq_a(x))) if self.wq is None else self.wq(x)
        q = q.view(T, H, dn + dr)
        kv_a = self.wkv_a(x)
        kv = self.wkv_b(self.kv_norm(kv_a[:, :c.kv_lora_rank])).view(T, H, dn + dv)
        if _assemble_kernel_ok(q, kv, kv_a, positions, self.rope, dn, dr, dv, c.kv_lora_rank):
            # one kernel: rotary embedding of q_pe and k_pe, [nope | pe] assembly of queries and keys, contiguous values
            qf, kf, v = _MLAAssembleFn.apply(q, kv, kv_a[:, c.kv_lora_rank:], self.rope.cache, positions, dn, dr, dv)
        else:
            q_pe = self.rope(q[:, :, dn:], positions)
            k_pe = self.rope(kv_a[:, c.kv_lora_rank:].reshape(T, 1, dr), positions)
            qf = torch.cat([q[:, :, :dn], q_pe], dim=-1)
            kf = torch.cat([kv[:, :, :dn], k_pe.expand(T, H, dr)], dim=-1)
            v = kv[:, :, dn:]
        ctx = ctx or AttentionContext()
        if ctx.kv_cache is not None:
            # incremental decoding: the assembled per-head keys and values are cached
            from .attention import cached_attention

            o = cached_attention(self, qf, kf, v.contiguous(), ctx.kv_cache, self.scale)
        elif ctx.cp is not None:
            from torchtitan_b200.parallel.context_parallel import cp_attention

            o = cp_attention(qf, kf, v, ctx, scale=self.scale, window=None, sinks=None)
        else:
            o = OF.attention(qf, kf, v, scale=self.scale, causal=True, doc_ids=ctx.doc_ids, kv_first=ctx.kv_first)
        y = self.wo(o.reshape(T, H * dv))
        if tp is not None:
            return tp_ops.reduce_scatter_rows(y, tp) if tp.sequence_parallel else tp_ops.all_reduce(y, tp)
        return y
