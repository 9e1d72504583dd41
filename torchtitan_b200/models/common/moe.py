"""Mixture of experts: token-choice top-k router, grouped SwiGLU experts, optional shared experts.

Parameter names follow the reference so checkpoints interoperate:
``moe.router.gate.weight``, ``moe.routed_experts.inner_experts.{w1_EFD,w2_EDF,w3_EFD}``,
``moe.shared_experts.{w1,w2,w3}.weight`` and the persistent buffer ``moe.expert_bias_E``
(torchtitan/models/common/moe.py:35-468).

Data flow for one layer (local experts or expert parallel):

    gate GEMM (fp32) -> softmax/sigmoid -> top-k (+bias, group limits) -> histogram
    -> dispatch: rows sorted expert-major (and exchanged over the ep group)
    -> grouped GEMMs: silu(x w1^T) * (x w3^T) -> w2
    -> combine: rows return to their owners, are scaled by the gate value in fp32 and
       summed per token (deterministic index_add order).

Load balancing is auxiliary-loss free: ``tokens_per_expert_E`` counts routed tokens and the
optimizer pre-hook turns it into an update of ``expert_bias_E`` (components/optimizer.py).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200.ops import functional as OF
from torchtitan_b200.ops import reference as ref

from .layers import FeedForward, Linear, TPContext
from .module import InitSpec, Module, set_init

__all__ = ["MoE", "GroupedExperts", "TokenChoiceTopKRouter", "RoutedExperts", "grouped_mm"]


# ----------------------------------------------------------------------------
# grouped GEMM front-end
# ----------------------------------------------------------------------------
def _grouped_mm_loop(x: torch.Tensor, w_ekn: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """Reference path: ``out[rows of expert e] = x[rows] @ w[e]`` with ``w[e]`` of shape ``[K, N]``."""
    out = x.new_zeros(x.shape[0], w_ekn.shape[-1])
    bounds = [0] + offs.tolist()
    pieces = []
    for e in range(w_ekn.shape[0]):
        a, b = bounds[e], bounds[e + 1]
        pieces.append(x[a:b] @ w_ekn[e])
    if bounds[-1] < x.shape[0]:
        pieces.append(out[bounds[-1]:])
    return torch.cat(pieces, dim=0)


def grouped_mm(x: torch.Tensor, w_ekn: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """Rows of ``x`` are grouped by expert (``offs`` = int32 cumulative row counts)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and hasattr(torch, "_grouped_mm"):
        return torch._grouped_mm(x, w_ekn, offs=offs)
    return _grouped_mm_loop(x, w_ekn, offs)


class GroupedExperts(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        hidden_dim: int = 0
        num_experts: int = 0
        init_std: float = 0.02
        out_init_std: float = 0.02
        quant_recipe: str | None = None
        """``mxfp8`` / ``float8_rowwise``: block-scaled fp8 numerics for the three grouped GEMMs
        (set by the grouped-experts quantisation converters)."""

    def __init__(self, config: "GroupedExperts.Config", **_):
        super().__init__(config)
        c = config
        self.num_experts = c.num_experts
        self.quant_recipe = c.quant_recipe
        self.w1_EFD = nn.Parameter(torch.empty(c.num_experts, c.hidden_dim, c.dim))
        self.w2_EDF = nn.Parameter(torch.empty(c.num_experts, c.dim, c.hidden_dim))
        self.w3_EFD = nn.Parameter(torch.empty(c.num_experts, c.hidden_dim, c.dim))
        set_init(self.w1_EFD, InitSpec(kind="trunc_normal", std=c.init_std))
        set_init(self.w3_EFD, InitSpec(kind="trunc_normal", std=c.init_std))
        set_init(self.w2_EDF, InitSpec(kind="trunc_normal", std=c.out_init_std))
        for p in (self.w1_EFD, self.w2_EDF, self.w3_EFD):
            p._is_expert = True

    def shard_experts_(self, ep_size: int, ep_rank: int) -> None:
        """Expert parallel: keep experts ``[r*E/ep, (r+1)*E/ep)``."""
        E = self.num_experts
        if E % ep_size:
            raise ValueError(f"num_experts={E} must divide by ep={ep_size}")
        from torchtitan_b200.parallel import sharding as shd

        self.sharding = shd.expert_parallel()
        for name, layout in self.sharding.state_shardings.items():
            new = shd.shard_parameter(getattr(self, name), layout.on("ep"), ep_size, ep_rank)
            new._is_expert = True
            setattr(self, name, new)
        self.num_experts = E // ep_size

    def shard_tp_(self, tp: TPContext) -> None:
        """Expert tensor parallel (EP off): hidden dim split, w1/w3 on dim 1, w2 on dim 2."""
        from torchtitan_b200.parallel import sharding as shd

        self.sharding = shd.expert_tensor_parallel(tp.sequence_parallel)
        for name, layout in self.sharding.state_shardings.items():
            place = layout.on("tp")
            p = getattr(self, name)
            if p.shape[place.dim] % tp.size:
                raise ValueError("expert hidden dim must divide by tp")
            new = shd.shard_parameter(p, place, tp.size, tp.rank)
            new._is_expert = True
            setattr(self, name, new)

    def native_ok(self, x: torch.Tensor) -> bool:
        """The tcgen05 grouped GEMMs need bf16 CUDA rows and tile-friendly expert shapes."""
        from torchtitan_b200.ops import moe_ops

        return OF.settings.gemm == "tcgen05" and moe_ops.native_ok(x, self.w1_EFD.shape[2], self.w1_EFD.shape[1])

    def forward_padded(self, x: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
        """``x[R, dim]`` in the padded expert-major layout of ``ops.moe_ops`` (``offs[E_local + 1]``)."""
        from torchtitan_b200.ops import moe_ops

        if self.quant_recipe:
            return self._quant_forward(x, offs, padded=True)
        return moe_ops.grouped_swiglu_experts(x, self.w1_EFD, self.w3_EFD, self.w2_EDF, offs)

    def _quant_forward(self, x: torch.Tensor, offs: torch.Tensor, padded: bool) -> torch.Tensor:
        from torchtitan_b200.components.quantization.grouped import quant_grouped_linear as qgl

        r = self.quant_recipe
        h = qgl(x, self.w1_EFD, offs, r, padded)
        u = qgl(x, self.w3_EFD, offs, r, padded)
        a = (F.silu(h.float()) * u.float()).to(x.dtype)
        return qgl(a, self.w2_EDF, offs, r, padded)

    def forward(self, x: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
        """``x[N, dim]`` rows sorted by local expert; ``offs[E_local]`` cumulative counts (int32)."""
        if self.quant_recipe:
            return self._quant_forward(x, offs, padded=False)
        h = grouped_mm(x, self.w1_EFD.transpose(-2, -1), offs)
        u = grouped_mm(x, self.w3_EFD.transpose(-2, -1), offs)
        a = (F.silu(h.float()) * u.float()).to(x.dtype)
        return grouped_mm(a, self.w2_EDF.transpose(-2, -1), offs)


class TokenChoiceTopKRouter(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        num_experts: int = 0
        num_expert_groups: int | None = None
        num_limited_groups: int | None = None
        top_k: int = 1
        score_func: Literal["softmax", "sigmoid"] = "sigmoid"
        route_norm: bool = False
        route_scale: float = 1.0
        gate_init_std: float = 0.02
        gate_bias: bool = False
        _debug_force_load_balance: bool = False

    def __init__(self, config: "TokenChoiceTopKRouter.Config", **_):
        super().__init__(config)
        c = config
        self.gate = Linear(Linear.Config(in_features=c.dim, out_features=c.num_experts, init_std=c.gate_init_std,
                                         bias=c.gate_bias))
        self.gate.weight._replicated_over_tp = True
        if self.gate.bias is not None:
            self.gate.bias._replicated_over_tp = True
        self.num_experts, self.top_k = c.num_experts, c.top_k

    def forward(self, x: torch.Tensor, expert_bias: torch.Tensor | None):
        c = self.config
        # the gate runs in fp32 (parity: fp32 autocast of the router GEMM)
        logits = F.linear(x.float(), self.gate.weight.float(),
                          None if self.gate.bias is None else self.gate.bias.float())
        grouped = bool(c.num_expert_groups and c.num_limited_groups and c.num_expert_groups > 1)
        if logits.is_cuda and not grouped and not c._debug_force_load_balance and c.num_experts <= 512 and c.top_k <= 16:
            # fused sm_100a router: scores, biased top-k, renormalisation, scaling and histogram in one kernel
            from torchtitan_b200.ops import moe_ops

            return moe_ops.router_topk(logits, expert_bias, c.top_k, c.score_func, c.route_norm, c.route_scale)
        scores = torch.softmax(logits, dim=-1) if c.score_func == "softmax" else torch.sigmoid(logits)
        with torch.no_grad():
            if c._debug_force_load_balance:
                T = x.shape[0]
                base = torch.arange(T, device=x.device)[:, None] * c.top_k + torch.arange(c.top_k, device=x.device)
                sel = base % c.num_experts
                counts = torch.zeros(c.num_experts, dtype=torch.float32, device=x.device)
                counts.scatter_add_(0, sel.reshape(-1), torch.ones(sel.numel(), device=x.device))
            else:
                _, sel, counts = ref.router_topk(logits.detach(), c.top_k, c.score_func, expert_bias, False, 1.0,
                                                 c.num_expert_groups, c.num_limited_groups)
        top = scores.gather(-1, sel)
        if c.route_norm:
            top = top / (top.sum(dim=-1, keepdim=True) + 1e-20)
        top = top * c.route_scale
        return top, sel, counts


class RoutedExperts(Module):
    """Dispatch -> experts -> combine.  The dispatcher is chosen by the parallel plan."""

    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        inner_experts: GroupedExperts.Config = field(default_factory=GroupedExperts.Config)

    def __init__(self, config: "RoutedExperts.Config", *, top_k: int = 1, **_):
        super().__init__(config)
        self.inner_experts = config.inner_experts.build()
        self.top_k = top_k
        self.ep = None  # parallel.expert_parallel.EPContext

    def forward(self, x: torch.Tensor, top_scores: torch.Tensor, selected: torch.Tensor,
                counts: torch.Tensor) -> torch.Tensor:
        T, D = x.shape
        K = selected.shape[1]
        if self.ep is None and self.inner_experts.native_ok(x):
            from torchtitan_b200.ops import moe_ops

            dest, offs, cap = moe_ops.padded_layout(selected, counts)
            xp = moe_ops.permute_rows(x, dest, cap)
            yp = self.inner_experts.forward_padded(xp, offs)
            return moe_ops.combine_rows(yp, dest, top_scores)
        nv = getattr(self.ep, "nvlink", None) if self.ep is not None else None
        if nv is not None and self.inner_experts.native_ok(x):
            from torchtitan_b200.parallel.ep_nvlink import ep_experts_nvlink

            return ep_experts_nvlink(nv, self.inner_experts, x, top_scores, selected, counts)
        flat = selected.reshape(-1).long()
        order = torch.argsort(flat, stable=True)  # slots sorted expert-major
        token_idx = order // K
        rows = x.index_select(0, token_idx)
        if self.ep is not None:
            from torchtitan_b200.parallel.expert_parallel import ep_experts

            y = ep_experts(self.ep, self.inner_experts, rows, counts)
        else:
            offs = torch.cumsum(counts, 0).to(torch.int32)
            y = self.inner_experts(rows, offs)
        w = top_scores.reshape(-1).index_select(0, order).float()
        y = y.float() * w[:, None]
        out = torch.zeros(T, D, dtype=torch.float32, device=x.device)
        out.index_add_(0, token_idx, y)
        return out.to(x.dtype)


class MoE(Module):
    is_moe_layer = True

    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        hidden_dim: int = 0
        num_experts: int = 8
        top_k: int = 1
        router: TokenChoiceTopKRouter.Config = field(default_factory=TokenChoiceTopKRouter.Config)
        routed_experts: RoutedExperts.Config = field(default_factory=RoutedExperts.Config)
        load_balance_coeff: float | None = 1e-3
        shared_hidden_dim: int = 0
        shared_experts: FeedForward.Config | None = None
        shared_expert_gate: bool = False
        """Scale the shared experts' output by ``sigmoid(x w_gate)`` per token (Qwen3.5 MoE)."""

    def __init__(self, config: "MoE.Config", **_):
        super().__init__(config)
        c = config
        c.router.dim, c.router.num_experts, c.router.top_k = c.dim, c.num_experts, c.top_k
        ie = c.routed_experts.inner_experts
        ie.dim, ie.hidden_dim, ie.num_experts = c.dim, c.hidden_dim, c.num_experts
        self.router = c.router.build()
        self.routed_experts = c.routed_experts.build(top_k=c.top_k)
        self.shared_experts = None
        if c.shared_hidden_dim:
            sc = c.shared_experts or FeedForward.Config()
            sc.dim, sc.hidden_dim = c.dim, c.shared_hidden_dim
            self.shared_experts = sc.build()
        self.shared_gate = None
        if c.shared_expert_gate and self.shared_experts is not None:
            self.shared_gate = Linear(Linear.Config(in_features=c.dim, out_features=1, init_std=0.02))
            self.shared_gate.weight._replicated_over_tp = True
        self.load_balance_coeff = c.load_balance_coeff
        self.num_experts = c.num_experts
        if c.load_balance_coeff:
            self.register_buffer("expert_bias_E", torch.zeros(c.num_experts, dtype=torch.float32), persistent=True)
        else:
            self.expert_bias_E = None
        self.register_buffer("tokens_per_expert_E", torch.zeros(c.num_experts, dtype=torch.float32), persistent=False)

    # names used by the optimizer hook
    @property
    def expert_bias(self):
        return self.expert_bias_E

    @property
    def tokens_per_expert(self):
        return self.tokens_per_expert_E

    def init_buffers(self, device=None) -> None:
        dev = device if device is not None else self.tokens_per_expert_E.device
        if str(dev) == "meta":
            return
        self.tokens_per_expert_E = torch.zeros(self.num_experts, dtype=torch.float32, device=dev)
        if self.load_balance_coeff:
            self.expert_bias_E = torch.zeros(self.num_experts, dtype=torch.float32, device=dev)
        super().init_buffers(device)

    def shard_tp_(self, tp: TPContext) -> None:
        """Tensor parallel.  Without expert parallelism the experts are split on the hidden dim,
        tokens are gathered over tp inside the layer and the output is a partial sum.  With expert
        parallelism the layer works on this rank's sequence shard (tokens stay split over tp) and
        shared experts / router are replicated."""
        self.tp = tp
        if self.routed_experts.ep is None:
            self.routed_experts.inner_experts.shard_tp_(tp)
            if self.shared_experts is not None:
                self.shared_experts.w13.shard_("colwise", tp)
                self.shared_experts.w2.shard_("rowwise", tp)
                self.shared_experts.hidden_dim //= tp.size
        else:
            if not tp.sequence_parallel:
                raise ValueError("expert parallel + tensor parallel requires sequence parallelism")
            if self.shared_experts is not None:
                for p in self.shared_experts.parameters():
                    p._replicated_over_tp = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tp = getattr(self, "tp", None)
        gather = tp is not None and self.routed_experts.ep is None
        if gather:
            from torchtitan_b200.parallel import sharding as shd

            plan = self.routed_experts.inner_experts.sharding
            x = shd.redistribute(x, plan.in_src_shardings["x"].on("tp"), plan.in_dst_shardings["x"].on("tp"), tp)
        top, sel, counts = self.router(x, self.expert_bias_E)
        with torch.no_grad():
            self.tokens_per_expert_E.add_(counts)
        out = self.routed_experts(x, top, sel, counts)
        if self.shared_experts is not None:
            se = self.shared_experts
            shared = OF.swiglu_linear(se.w13(x), se.w2.weight)
            if self.shared_gate is not None:
                shared = shared * torch.sigmoid(self.shared_gate(x).float()).to(shared.dtype)
            out = out + shared
        if gather:
            return shd.redistribute(out, plan.out_src_shardings.on("tp"), plan.out_dst_shardings.on("tp"), tp)
        return out
