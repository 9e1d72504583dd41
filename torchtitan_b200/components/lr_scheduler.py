"""Warmup-stable-decay learning-rate schedule.

Multiplier at 0-indexed scheduler step ``s`` (parity:
torchtitan/components/optimizer/lr_scheduler.py:100-184): linear warmup
``(s+1)/warmup``; stable phase 1; decay over ``round(total*decay_ratio)`` steps (or
all remaining steps) with ``linear`` / ``sqrt`` / ``cosine`` shape, floored at
``min_lr_factor``.  The schedule has one extra virtual step so that the last real
step does not reach a zero learning rate.  State is only ``last_epoch``; the rate is
re-derived on load so a job may resume with a different ``steps``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Literal

from torchtitan_b200.config import Configurable

__all__ = ["LRSchedulersContainer", "wsd_multiplier"]


def wsd_multiplier(step: int, *, warmup_steps: int, total_steps: int, decay_ratio: float | None,
                   decay_type: str, min_lr_factor: float) -> float:
    warmup_steps = min(warmup_steps, total_steps)
    if decay_ratio is not None:
        decay_steps = min(round(total_steps * decay_ratio), total_steps - warmup_steps)
    else:
        decay_steps = total_steps - warmup_steps
    stable_steps = total_steps + 1 - warmup_steps - decay_steps
    if step < warmup_steps:
        return (step + 1) / warmup_steps
    if step < warmup_steps + stable_steps:
        return 1.0
    progress = (step + 1 - warmup_steps - stable_steps) / max(1, decay_steps)
    progress = min(progress, 1.0)
    if decay_type == "linear":
        value = 1.0 - progress
    elif decay_type == "sqrt":
        value = 1.0 - math.sqrt(progress)
    elif decay_type == "cosine":
        value = 0.5 * (1.0 + math.cos(math.pi * progress))
    else:
        raise ValueError(f"unknown decay type {decay_type}")
    return min_lr_factor + (1.0 - min_lr_factor) * value


class LRSchedulersContainer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        warmup_steps: int = 200
        total_steps: int | None = None
        decay_ratio: float | None = None
        decay_type: Literal["linear", "sqrt", "cosine"] = "linear"
        min_lr_factor: float = 0.0

    def __init__(self, config: "LRSchedulersContainer.Config", *, optimizers, training_steps: int, **_):
        self.config = config
        self.optimizers = optimizers
        self.total_steps = config.total_steps if config.total_steps is not None else training_steps
        if config.decay_ratio is not None and not 0.0 <= config.decay_ratio <= 1.0:
            raise ValueError("lr_scheduler.decay_ratio must be within [0, 1]")
        self.last_epoch = 0
        self.base_lrs = [g["lr"] for g in optimizers.param_groups]
        for g in optimizers.param_groups:
            g.setdefault("initial_lr", g["lr"])
        self._apply()

    def multiplier(self, step: int | None = None) -> float:
        c = self.config
        return wsd_multiplier(self.last_epoch if step is None else step, warmup_steps=c.warmup_steps,
                              total_steps=self.total_steps, decay_ratio=c.decay_ratio, decay_type=c.decay_type,
                              min_lr_factor=c.min_lr_factor)

    def _apply(self) -> None:
        m = self.multiplier()
        for g, base in zip(self.optimizers.param_groups, self.base_lrs):
            g["lr"] = base * m

    def step(self) -> None:
        self.last_epoch += 1
        self._apply()

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizers.param_groups]

    def get_metrics(self) -> dict[str, float]:
        lrs = self.get_last_lr()
        name = self.optimizers.optimizer_name
        if len(lrs) == 1:
            return {f"lr/{name}": lrs[0]}
        return {f"lr/{name}/{i}": v for i, v in enumerate(lrs)}

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch}

    def load_state_dict(self, sd: dict) -> None:
        self.last_epoch = int(sd["last_epoch"])
        self._apply()
