"""Optimizer container over the sharded engines.

The optimizer state lives in the engines' flat fp32 shards
(:mod:`torchtitan_b200.parallel.fsdp`); this container owns the hyper-parameters,
the parameter-group assignment (regex on the FQN, first match wins), the gradient
clipping coefficient and the checkpoint view.  ``implementation`` keeps the
reference's names: ``fused`` (our flat AdamW kernel, fp32 moments) and
``fused_opt_states_bf16`` (bf16 moments, fp32 math); ``foreach`` / ``for-loop`` map to
the same kernel.  Optimizers: ``Adam``, ``AdamW`` and ``DistMuon`` (matrix parameters; see
:mod:`torchtitan_b200.parallel.muon`), mixed per param group.
Parity: torchtitan/components/optimizer/optimizer.py:41-526.

Non-finite protection.  The clip coefficient is a device scalar.  When the loss or
the gradient norm is not finite the coefficient becomes NaN, the AdamW kernel then
leaves parameters and moments untouched, and the host raises at its next
synchronisation point -- no device-side assert is involved.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any, Literal

import torch
import torch.distributed as dist

from torchtitan_b200.config import Configurable
from torchtitan_b200.ops import optim as optim_ops

__all__ = ["ParamGroupConfig", "OptimizersContainer", "clip_grad_norm_", "MoEBiasUpdater"]


@dataclass(kw_only=True, slots=True)
class ParamGroupConfig:
    pattern: str = ".*"
    optimizer_name: str = "AdamW"
    optimizer_kwargs: dict[str, Any] = field(default_factory=dict)


class OptimizersContainer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        name: str = "AdamW"
        lr: float = 8e-4
        beta1: float = 0.9
        beta2: float = 0.95
        eps: float = 1e-8
        weight_decay: float = 0.1
        implementation: Literal["for-loop", "foreach", "fused", "fused_opt_states_bf16"] = "fused"
        param_groups: list[ParamGroupConfig] = field(default_factory=list)
        optimizer_factory_kwargs_by_name: dict[str, dict[str, Any]] = field(default_factory=dict)

    def __init__(self, config: "OptimizersContainer.Config", *, engines: list, **_):
        self.config = config
        self.engines = list(engines)
        c = config
        known = ("AdamW", "Adam", "DistMuon")
        if c.name not in known:
            raise NotImplementedError(f"optimizer '{c.name}' is not available (have {', '.join(known)})")
        self.optimizer_name = c.name

        def group_for(name: str, kwargs: dict) -> dict:
            """Hyper-parameters of one param group: the optimizer's defaults, the container's
            fields, the factory kwargs of that optimizer, then the group's own kwargs."""
            if name not in known:
                raise NotImplementedError(f"optimizer '{name}' is not available (have {', '.join(known)})")
            if name == "DistMuon":
                from torchtitan_b200.parallel.muon import MUON_DEFAULTS

                g = dict(MUON_DEFAULTS, lr=c.lr, weight_decay=c.weight_decay)
            else:
                g = dict(lr=c.lr, betas=(c.beta1, c.beta2), eps=c.eps,
                         weight_decay=c.weight_decay if name == "AdamW" else 0.0)
            g.update(c.optimizer_factory_kwargs_by_name.get(name, {}))
            kw = dict(kwargs)
            kw.pop("foreach", None)   # accepted for recipe compatibility; one implementation here
            if "betas" in kw:
                kw["betas"] = tuple(kw["betas"])
            g.update(kw)
            g["optimizer_name"] = name
            return g

        self.param_groups: list[dict] = []
        patterns = []
        for pg in c.param_groups:
            re.compile(pg.pattern)
            g = group_for(pg.optimizer_name, pg.optimizer_kwargs)
            g["pattern"] = pg.pattern
            self.param_groups.append(g)
            patterns.append(pg.pattern)
        default = group_for(c.name, {})
        default["pattern"] = None
        self.param_groups.append(default)
        self.group_members: list[list[str]] = [[] for _ in self.param_groups]
        for e in self.engines:
            members = e.assign_groups(patterns)
            for i, m in enumerate(members):
                self.group_members[i].extend(m)
        for pat, mem in zip(patterns, self.group_members):
            if not mem:
                raise ValueError(f"optimizer param group pattern '{pat}' matched no parameter")
        self._grad_scale: torch.Tensor | float = 1.0
        self._pre_hooks = []

    def register_step_pre_hook(self, fn) -> None:
        self._pre_hooks.append(fn)

    def set_grad_scale(self, scale) -> None:
        self._grad_scale = scale

    def step(self) -> None:
        for h in self._pre_hooks:
            h(self)
        for e in self.engines:
            e.adamw_step(self.param_groups, self._grad_scale)
        self._grad_scale = 1.0

    def zero_grad(self, set_to_none: bool = True) -> None:
        for e in self.engines:
            e.zero_grad()

    # -- checkpoint view -----------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        from torchtitan_b200.components.checkpoint import engine_optimizer_state

        out: dict[str, Any] = {}
        for e in self.engines:
            out.update(engine_optimizer_state(e, self.param_groups))
        return out

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        from torchtitan_b200.components.checkpoint import load_engine_optimizer_state

        for e in self.engines:
            load_engine_optimizer_state(e, sd, self.param_groups)


@torch.no_grad()
def clip_grad_norm_(engines: list, max_norm: float, pdims, *, loss_finite: torch.Tensor | None = None,
                    optimizers: OptimizersContainer | None = None) -> torch.Tensor:
    """Global L2 norm over every gradient shard of every engine, and the clip scale.

    Squared norms are summed over the sharding group, the tensor-parallel group
    (replicated parameters counted once), the pipeline group and, for expert
    parameters, their own sharding group (parity: torchtitan/distributed/utils.py:594-740).
    The scale ``min(1, max_norm/(norm+1e-6))`` is handed to the optimizer, which fuses
    it into the update instead of rewriting the gradients.
    """
    dev = engines[0].device
    total = torch.zeros((), dtype=torch.float32, device=dev)
    for e in engines:
        e.finalize_grads()
        ss = e.local_sumsq()
        tp = pdims.tp if pdims is not None else 1
        total += ss[0] / max(tp, 1) + ss[1]
    if pdims is not None and pdims.world_size > 1 and dist.is_initialized():
        # every rank holds a disjoint set of gradient elements (after the division of the
        # tp-replicated part), except ranks that only differ in dp_replicate
        dist.all_reduce(total, group=dist.group.WORLD)
        if pdims.dp_replicate > 1:
            total /= pdims.dp_replicate
    norm = total.sqrt()
    scale = optim_ops.clip_coefficient(norm, max_norm) if max_norm and max_norm > 0 else torch.ones_like(norm)
    bad = ~torch.isfinite(norm)
    if loss_finite is not None:
        bad = bad | ~loss_finite.to(torch.bool)
    scale = torch.where(bad, torch.full_like(scale, float("nan")), scale)
    if optimizers is not None:
        optimizers.set_grad_scale(scale.reshape(1))
    return norm


class MoEBiasUpdater:
    """Auxiliary-loss-free load balancing, run before each optimizer step.

    ``delta = coeff * sign(mean(c) - c)``, zero-meaned, added to the routing bias;
    the token counter is then cleared (parity: optimizer.py:402-526).  Counts are
    summed over the ``loss`` mesh (and over tp when experts are parallel).
    """

    def __init__(self, model_parts, pdims, full_ac: bool = False):
        self.moes = [m for part in model_parts for m in part.modules() if getattr(m, "is_moe_layer", False)
                     and m.load_balance_coeff]
        self.pdims = pdims
        self.full_ac = full_ac

    @torch.no_grad()
    def __call__(self, _opt=None) -> None:
        if not self.moes:
            return
        counts = torch.stack([m.tokens_per_expert for m in self.moes])
        if self.full_ac:
            counts = counts / 2  # recomputation routes every token twice
        if self.pdims is not None and dist.is_initialized():
            if self.pdims.ep_enabled and self.pdims.tp_enabled:
                dist.all_reduce(counts, group=self.pdims.group("tp"))
            g = self.pdims.group("loss")
            if g is not None:
                dist.all_reduce(counts, group=g)
        for m, c in zip(self.moes, counts):
            delta = m.load_balance_coeff * torch.sign(c.mean() - c)
            delta = delta - delta.mean()
            m.expert_bias.add_(delta)
            m.tokens_per_expert.zero_()
