"""Gated DeltaNet linear attention (Qwen3.5 / Qwen3-Next).

Per head, with L2-normalised ``q, k`` and ``q`` scaled by ``dk^-1/2``, the state ``S[dk, dv]`` follows

    S_t = exp(g_t) S_{t-1} + k_t (beta_t (v_t - k_t^T exp(g_t) S_{t-1}))^T,      o_t = q_t^T S_t

with ``g_t = -exp(A_log) softplus(a_t + dt_bias) <= 0`` and ``beta_t = sigmoid(b_t)``.  q, k, v first
pass a depthwise causal convolution (kernel 4) + SiLU; the output passes a gated RMSNorm
``silu(z) * w * norm(o)`` and the output projection.  State and convolution restart at document
boundaries.  ``chunk_gated_delta_rule`` is the chunked (matmul-rich) evaluation of the same
recurrence, ``recurrent_gated_delta_rule`` the step-by-step oracle.
Parity: torchtitan/models/qwen3_5/gdn.py:45-539 (which calls the fla Triton kernels).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200.models.common.attention import AttentionContext
from torchtitan_b200.models.common.layers import Linear, RMSNorm
from torchtitan_b200.models.common.module import InitSpec, Module, set_init
from torchtitan_b200.parallel import tp_ops

__all__ = ["GatedDeltaNet", "chunk_gated_delta_rule", "recurrent_gated_delta_rule", "causal_conv_silu"]

_RESET = -1.0e3  # log-decay placed on the first token of a document: exp() of it is zero in fp32


def _l2norm(x: torch.Tensor) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def recurrent_gated_delta_rule(q, k, v, g, beta):
    """``q, k [T, H, dk]``, ``v [T, H, dv]``, ``g, beta [T, H]`` -> ``o [T, H, dv]`` (fp32 loop)."""
    T, H, dk = q.shape
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q = _l2norm(q) * dk ** -0.5
    k = _l2norm(k)
    S = q.new_zeros(H, dk, v.shape[-1])
    out = []
    for t in range(T):
        S = S * torch.exp(g[t])[:, None, None]
        mem = torch.einsum("hk,hkv->hv", k[t], S)
        delta = (v[t] - mem) * beta[t][:, None]
        S = S + torch.einsum("hk,hv->hkv", k[t], delta)
        out.append(torch.einsum("hk,hkv->hv", q[t], S))
    return torch.stack(out)


def chunk_gated_delta_rule(q, k, v, g, beta, chunk: int = 64, *, initial_state=None, return_state: bool = False):
    """Chunked evaluation of the gated delta rule (same signature as the recurrent oracle).  ``initial_state``
    ``[H, dk, dv]`` continues an earlier call (incremental decoding); ``return_state`` also returns the state after
    the last token (padding rows have zero keys, values and gates, so they leave it unchanged)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    dt = v.dtype
    q, k, v, g, beta = (t.float().transpose(0, 1) for t in (q, k, v, g, beta))   # [H, T, ...]
    q = _l2norm(q) * dk ** -0.5
    k = _l2norm(k)
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    N = (T + pad) // chunk
    q, k, v = (t.reshape(H, N, chunk, -1) for t in (q, k, v))
    g, beta = g.reshape(H, N, chunk), beta.reshape(H, N, chunk)
    v_beta, k_beta = v * beta[..., None], k * beta[..., None]
    gc = g.cumsum(-1)
    diff = gc[..., :, None] - gc[..., None, :]
    lower = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    decay = torch.exp(diff.masked_fill(~lower, float("-inf")))          # zero above the diagonal
    strict = lower & ~torch.eye(chunk, dtype=torch.bool, device=q.device)
    a = -(k_beta @ k.transpose(-1, -2) * decay).masked_fill(~strict, 0.0)
    # (I - A)^-1 by forward substitution over the rows of the strictly lower triangle
    rows = [a[..., 0, :]]
    for i in range(1, chunk):
        prev = torch.stack(rows, dim=-2)                                  # [.., i, C]
        rows.append(a[..., i, :] + (a[..., i, :i, None] * prev).sum(-2))
    a = torch.stack(rows, dim=-2) + torch.eye(chunk, device=q.device)
    value = a @ v_beta
    k_cum = a @ (k_beta * torch.exp(gc)[..., None])
    S = q.new_zeros(H, dk, dv) if initial_state is None else initial_state.float()
    outs = []
    for i in range(N):
        qi, ki, vi, gi = q[:, i], k[:, i], value[:, i], gc[:, i]
        attn = (qi @ ki.transpose(-1, -2) * decay[:, i]).masked_fill(~lower, 0.0)
        v_new = vi - k_cum[:, i] @ S
        inter = (qi * torch.exp(gi)[..., None]) @ S
        outs.append(inter + attn @ v_new)
        S = S * torch.exp(gi[:, -1])[:, None, None] + (ki * torch.exp(gi[:, -1:] - gi)[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=1).reshape(H, N * chunk, dv)[:, :T]
    if return_state:
        return o.transpose(0, 1).to(dt), S
    return o.transpose(0, 1).to(dt)


class _ConvSiluFn(torch.autograd.Function):
    """The convolution + SiLU as one kernel each way (``ops/csrc/conv.cu``): x is read once, the backward recomputes
    the pre-activation and returns dx and the fp32 weight gradient."""

    @staticmethod
    def forward(ctx, x, weight, positions):
        from torchtitan_b200.ops import ext
        from torchtitan_b200.ops.functional import _count

        w32 = weight.detach().float().contiguous()
        pos = None if positions is None else positions.to(torch.int64).contiguous()
        ctx.save_for_backward(x, w32, pos if pos is not None else torch.empty(0))
        ctx.has_pos = pos is not None
        ctx.weight = weight
        _count()
        return ext.require().conv_silu_fwd(x, w32, pos)

    @staticmethod
    def backward(ctx, dy):
        from torchtitan_b200.ops import ext
        from torchtitan_b200.ops.functional import _count, _deliver_wgrad

        x, w32, pos = ctx.saved_tensors
        _count()
        dx, dw = ext.require().conv_silu_bwd(x, w32, pos if ctx.has_pos else None, dy.contiguous())
        w = ctx.weight
        return dx, _deliver_wgrad(w, dw.to(w.dtype)) if w.requires_grad else None, None


def _conv_kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    from torchtitan_b200.ops import ext

    return (x.is_cuda and x.dim() == 2 and x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float32)
            and weight.shape[-1] <= 4 and x.shape[1] % (8 if x.dtype == torch.bfloat16 else 4) == 0 and ext.available())


def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, positions: torch.Tensor | None) -> torch.Tensor:
    """Depthwise causal convolution over tokens + SiLU.  ``x [T, C]``, ``weight [C, W]``; taps that
    would reach before the start of the token's document (``positions``) contribute nothing."""
    if _conv_kernel_ok(x, weight):
        return _ConvSiluFn.apply(x, weight, positions)
    T, C = x.shape
    W = weight.shape[-1]
    y = x * weight[:, W - 1].to(x.dtype)
    for j in range(1, W):
        shifted = F.pad(x[:-j], (0, 0, j, 0)) if j < T else torch.zeros_like(x)
        if positions is not None:
            shifted = shifted * (positions >= j).to(x.dtype)[:, None]
        y = y + shifted * weight[:, W - 1 - j].to(x.dtype)
    return F.silu(y)


class GatedDeltaNet(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        n_key_heads: int = 0
        n_value_heads: int = 0
        key_head_dim: int = 128
        value_head_dim: int = 128
        conv_kernel_size: int = 4
        norm_eps: float = 1e-6
        init_std: float = 0.02
        out_init_std: float = 0.02
        chunk_size: int = 64
        # interface parity with attention configs (used by the parameter accounting)
        n_heads: int = 0
        n_kv_heads: int | None = None
        head_dim: int | None = None
        qk_norm: object | None = None
        use_sinks: bool = False
        wqkv: Linear.Config = field(default_factory=Linear.Config)
        wo: Linear.Config = field(default_factory=Linear.Config)

    def __init__(self, config: "GatedDeltaNet.Config", **_):
        super().__init__(config)
        c = config
        kd, vd = c.n_key_heads * c.key_head_dim, c.n_value_heads * c.value_head_dim
        L = Linear.Config
        self.in_proj_q = L(in_features=c.dim, out_features=kd, init_std=c.init_std).build()
        self.in_proj_k = L(in_features=c.dim, out_features=kd, init_std=c.init_std).build()
        self.in_proj_v = L(in_features=c.dim, out_features=vd, init_std=c.init_std).build()
        self.in_proj_z = L(in_features=c.dim, out_features=vd, init_std=c.init_std).build()
        self.in_proj_a = L(in_features=c.dim, out_features=c.n_value_heads, init_std=c.init_std).build()
        self.in_proj_b = L(in_features=c.dim, out_features=c.n_value_heads, init_std=c.init_std).build()
        self.conv_q = nn.Parameter(torch.empty(kd, c.conv_kernel_size))
        self.conv_k = nn.Parameter(torch.empty(kd, c.conv_kernel_size))
        self.conv_v = nn.Parameter(torch.empty(vd, c.conv_kernel_size))
        bound = c.conv_kernel_size ** -0.5
        for p in (self.conv_q, self.conv_k, self.conv_v):
            set_init(p, InitSpec(kind="uniform", a=-bound, b=bound))
        self.A_log = nn.Parameter(torch.empty(c.n_value_heads))
        self.dt_bias = nn.Parameter(torch.empty(c.n_value_heads))
        set_init(self.A_log, InitSpec(kind="uniform", a=0.0, b=2.77))      # log of uniform(1, 16)
        set_init(self.dt_bias, InitSpec(kind="ones"))
        self.norm_weight = nn.Parameter(torch.empty(c.value_head_dim))
        set_init(self.norm_weight, InitSpec(kind="ones"))
        self.out_proj = L(in_features=vd, out_features=c.dim, init_std=c.out_init_std).build()
        self.tp = None
        for p in (self.A_log, self.dt_bias, self.norm_weight):
            p._replicated_over_tp = True

    def shard_(self, tp) -> None:
        """Tensor parallel: the layer runs replicated on the gathered sequence (its projections are small
        next to the MLP); all parameters are marked replicated."""
        self.tp = tp
        for p in self.parameters():
            p._replicated_over_tp = True
            # without sequence parallelism every rank runs the whole layer on the whole sequence
            p._tp_grad_complete_without_sp = True

    def forward(self, x: torch.Tensor, positions: torch.Tensor, ctx: AttentionContext | None = None,
                norm: RMSNorm | None = None) -> torch.Tensor:
        c = self.config
        if norm is not None:
            x = norm(x)
        tp = self.tp
        if tp is not None and tp.sequence_parallel:
            x = tp_ops.all_gather_rows(x, tp)
        T = x.shape[0]
        cache = ctx.kv_cache if ctx is not None else None
        packed = cache is None and ctx is not None and ctx.doc_ids is not None
        pos = positions if packed else None
        pq, pk, pv = self.in_proj_q(x), self.in_proj_k(x), self.in_proj_v(x)
        g = -torch.exp(self.A_log.float()) * F.softplus(self.in_proj_a(x).float() + self.dt_bias.float())
        beta = torch.sigmoid(self.in_proj_b(x).float())
        if packed:
            g = torch.where((positions == 0)[:, None], torch.full_like(g, _RESET), g)
        rep = c.n_value_heads // c.n_key_heads

        def mix(pq_, pk_, pv_, g_, beta_, state: dict | None):
            """Convolutions and the delta rule over one token range; ``state`` (incremental decoding) carries the last
            ``W - 1`` convolution inputs and the state matrix from the range before."""
            n = pq_.shape[0]

            def conv(p, w, name):
                if state is None:
                    return causal_conv_silu(p, w, pos)
                tail = state.get(name)
                full = p if tail is None else torch.cat([tail, p])
                state[name] = full[-(w.shape[-1] - 1):].detach().clone()
                return causal_conv_silu(full.contiguous(), w, None)[-n:]

            q = conv(pq_, self.conv_q, "q").view(n, c.n_key_heads, c.key_head_dim)
            k = conv(pk_, self.conv_k, "k").view(n, c.n_key_heads, c.key_head_dim)
            v = conv(pv_, self.conv_v, "v").view(n, c.n_value_heads, c.value_head_dim)
            if rep > 1:
                q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
            if state is None:
                return chunk_gated_delta_rule(q, k, v, g_, beta_, c.chunk_size)
            o_, state["S"] = chunk_gated_delta_rule(q, k, v, g_, beta_, c.chunk_size, initial_state=state.get("S"),
                                                    return_state=True)
            return o_

        if cache is None:
            o = mix(pq, pk, pv, g, beta, None)
        elif hasattr(cache, "caches"):          # several sequences in one pass: the token mixing is per sequence
            parts, r0 = [], 0
            for one, n in zip(cache.caches, cache.rows):
                sl = slice(r0, r0 + n)
                parts.append(mix(pq[sl], pk[sl], pv[sl], g[sl], beta[sl], one.state(self)))
                r0 += n
            o = torch.cat(parts)
        else:
            o = mix(pq, pk, pv, g, beta, cache.state(self))
        z = self.in_proj_z(x).view(T, c.n_value_heads, c.value_head_dim)
        of = o.float()
        of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + c.norm_eps) * self.norm_weight.float()
        y = self.out_proj((of * F.silu(z.float())).to(x.dtype).reshape(T, -1))
        if tp is not None and tp.sequence_parallel:
            S = T // tp.size
            return y[tp.rank * S:(tp.rank + 1) * S]
        return y
