"""LoRA: low-rank adapters on selected linears, everything else frozen.

``lora_converter`` rewrites the model config: every targeted ``Linear`` (or quantised linear)
config becomes the matching ``LoRA*`` config, whose module keeps the base weight frozen and adds
``lora_a [r, in]`` (Kaiming-uniform) and ``lora_b [out, r]`` (zeros) with output
``base(x) + (alpha / r) * (x lora_a^T) lora_b^T``.  The decoder then freezes every parameter
that is not an adapter.  Under tensor parallelism ``lora_b`` follows a column-parallel base and
``lora_a`` a row-parallel base; the other factor is replicated.
Parity: torchtitan/components/lora.py:23-235 (must come after quantisation converters).
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from torchtitan_b200.models.common.layers import Linear
from torchtitan_b200.models.common.module import InitSpec, set_init
from torchtitan_b200.ops import functional as OF

__all__ = ["lora_converter", "make_lora_class", "LORA_PARAM_PATTERN"]

LORA_PARAM_PATTERN = r"\.lora_[ab]$"
_DEFAULT_TARGETS = ("wqkv", "wo", "w13", "w2", "wq", "wq_b", "wkv_b")
_CLASSES: dict[type, type] = {}


def make_lora_class(parent: type) -> type:
    """``LoRA<Parent>``: a subclass of a Linear-like module with frozen base weight and adapters."""
    if parent in _CLASSES:
        return _CLASSES[parent]

    @dataclass(kw_only=True, slots=True)
    class Config(parent.Config):
        rank: int = 8
        alpha: float = 16.0

    class LoRALinear(parent):
        def __init__(self, config, **kw):
            super().__init__(config, **kw)
            c = config
            self.weight.requires_grad_(False)
            if self.bias is not None:
                self.bias.requires_grad_(False)
            self.lora_a = nn.Parameter(torch.empty(c.rank, self.in_features))
            self.lora_b = nn.Parameter(torch.empty(self.out_features, c.rank))
            set_init(self.lora_a, InitSpec(kind="uniform", a=-1.0 / math.sqrt(max(1, self.in_features)),
                                           b=1.0 / math.sqrt(max(1, self.in_features))))
            set_init(self.lora_b, InitSpec(kind="zeros"))
            self.scaling = c.alpha / c.rank

        def shard_(self, mode, tp):
            full_out, full_in = self.out_features, self.in_features
            super().shard_(mode, tp)
            self.weight.requires_grad_(False)
            if self.bias is not None:
                self.bias.requires_grad_(False)
            r = self.config.rank
            if mode == "colwise":
                rows = self.weight._tp_slices[1]
                nb = nn.Parameter(torch.empty(self.out_features, r, device=self.lora_b.device, dtype=self.lora_b.dtype))
                nb._tp_slices = (0, rows, (full_out, r))
                set_init(nb, self.lora_b._init_spec)
                self.lora_b = nb
                self.lora_a._replicated_over_tp = True
            else:
                k = self.in_features
                na = nn.Parameter(torch.empty(r, k, device=self.lora_a.device, dtype=self.lora_a.dtype))
                na._tp_slices = (1, [(tp.rank * k, (tp.rank + 1) * k)], (r, full_in))
                set_init(na, self.lora_a._init_spec)
                self.lora_a = na
                self.lora_b._replicated_over_tp = True

        def forward(self, x):
            base = super().forward(x)
            low = OF.linear(OF.linear(x.to(self.lora_a.dtype), self.lora_a), self.lora_b)
            return base + self.scaling * low

    Config.__qualname__ = f"LoRA{parent.__name__}.Config"
    LoRALinear.__name__ = LoRALinear.__qualname__ = f"LoRA{parent.__name__}"
    LoRALinear.Config = Config
    Config._owner = LoRALinear
    _CLASSES[parent] = LoRALinear
    return LoRALinear


def lora_converter(model_cfg, arg, job_config) -> int:
    """``arg``: ``rank=8,alpha=16,targets=wqkv+wo`` (all optional)."""
    from torchtitan_b200.components.quantization.utils import iter_linear_configs

    opts = dict(kv.split("=", 1) for kv in (arg or "").split(",") if "=" in kv)
    rank, alpha = int(opts.get("rank", 8)), float(opts.get("alpha", 16.0))
    targets = tuple(opts["targets"].split("+")) if "targets" in opts else _DEFAULT_TARGETS
    n = 0
    for fqn, owner, attr, lin in list(iter_linear_configs(model_cfg)):
        if attr not in targets or "lm_head" in fqn or "router" in fqn:
            continue
        parent = type(lin)._owner if hasattr(type(lin), "_owner") else Linear
        cls = make_lora_class(parent)
        kw = {f.name: getattr(lin, f.name) for f in dataclasses.fields(lin)}
        setattr(owner, attr, cls.Config(rank=rank, alpha=alpha, **kw))
        n += 1
    if n == 0:
        raise ValueError("the LoRA converter matched no Linear layer")
    model_cfg.trainable_param_pattern = LORA_PARAM_PATTERN
    return n
