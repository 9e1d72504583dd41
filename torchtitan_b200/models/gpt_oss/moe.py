"""GPT-OSS experts: fused gate/up projection with bias, clamped SwiGLU, down projection with bias.

``act(x) = min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)`` where the
gate ``g`` and the linear part ``u`` are the even and odd columns of the first projection.
Parameter names follow torchtitan/models/gpt_oss/moe.py:24-198
(``mlp1_weight [E, 2F, D]``, ``mlp1_bias [E, 2F]``, ``mlp2_weight [E, D, F]``, ``mlp2_bias [E, D]``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.module import InitSpec, Module, set_init

__all__ = ["GptOssExperts", "clamped_swiglu"]


def clamped_swiglu(x: torch.Tensor, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    g, u = x[..., ::2], x[..., 1::2]
    g = g.clamp(max=limit)
    u = u.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(alpha * g) * (u + 1)


class GptOssExperts(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        hidden_dim: int = 0
        num_experts: int = 0
        init_std: float = 0.02
        out_init_std: float = 0.02
        swiglu_limit: float = 7.0
        swiglu_alpha: float = 1.702

    def __init__(self, config: "GptOssExperts.Config", **_):
        super().__init__(config)
        c = config
        self.num_experts = c.num_experts
        self.mlp1_weight = nn.Parameter(torch.empty(c.num_experts, 2 * c.hidden_dim, c.dim))
        self.mlp1_bias = nn.Parameter(torch.empty(c.num_experts, 2 * c.hidden_dim))
        self.mlp2_weight = nn.Parameter(torch.empty(c.num_experts, c.dim, c.hidden_dim))
        self.mlp2_bias = nn.Parameter(torch.empty(c.num_experts, c.dim))
        set_init(self.mlp1_weight, InitSpec(kind="trunc_normal", std=c.init_std))
        set_init(self.mlp2_weight, InitSpec(kind="trunc_normal", std=c.out_init_std))
        set_init(self.mlp1_bias, InitSpec(kind="zeros"))
        set_init(self.mlp2_bias, InitSpec(kind="zeros"))
        for p in self.parameters():
            p._is_expert = True

    def native_ok(self, x: torch.Tensor) -> bool:
        return False  # biased experts with the clamped activation run on the library grouped GEMM

    def shard_experts_(self, ep_size: int, ep_rank: int) -> None:
        E = self.num_experts
        if E % ep_size:
            raise ValueError(f"num_experts={E} must divide by ep={ep_size}")
        n = E // ep_size
        for name in ("mlp1_weight", "mlp1_bias", "mlp2_weight", "mlp2_bias"):
            p = getattr(self, name)
            new = nn.Parameter(torch.empty(n, *p.shape[1:], device=p.device, dtype=p.dtype))
            new._tp_slices = (0, [(ep_rank * n, (ep_rank + 1) * n)], tuple(p.shape))
            new._is_expert = True
            set_init(new, p._init_spec)
            setattr(self, name, new)
        self.num_experts = n

    def shard_tp_(self, tp) -> None:
        raise NotImplementedError("GPT-OSS experts are sharded with expert parallelism, not expert tensor parallelism")

    def forward(self, x: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
        """``x[N, dim]`` rows sorted by local expert; ``offs[E_local]`` cumulative counts."""
        from torchtitan_b200.models.common.moe import grouped_mm

        c = self.config
        counts = torch.diff(offs.long(), prepend=offs.new_zeros(1).long())
        row_expert = torch.repeat_interleave(torch.arange(self.num_experts, device=x.device), counts,
                                             output_size=x.shape[0])
        h = grouped_mm(x, self.mlp1_weight.transpose(-2, -1), offs) + self.mlp1_bias[row_expert].to(x.dtype)
        a = clamped_swiglu(h.float(), c.swiglu_alpha, c.swiglu_limit).to(x.dtype)
        return grouped_mm(a, self.mlp2_weight.transpose(-2, -1), offs) + self.mlp2_bias[row_expert].to(x.dtype)
