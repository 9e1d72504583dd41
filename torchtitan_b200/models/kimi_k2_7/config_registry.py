"""Registered Kimi / Moonlight training configs (parity: torchtitan/models/kimi_k2_7/config_registry.py)."""

from __future__ import annotations

from torchtitan_b200.models.deepseek_v3.config_registry import _full, deepseek_v3_debugmodel
from torchtitan_b200.trainer import Trainer


def kimi_debugmodel() -> Trainer.Config:
    cfg = deepseek_v3_debugmodel()
    cfg.model.name, cfg.model.flavor = "kimi_k2_7", "debugmodel"
    return cfg


def kimi_moonlight() -> Trainer.Config:
    cfg = _full("moonlight", 2 * 8192, 8192, 4e-4, 10000, expert_parallel_degree=8)
    cfg.model.name = "kimi_k2_7"
    return cfg


def kimi_k2() -> Trainer.Config:
    cfg = _full("kimi_k2", 4 * 4096, 4096, 2e-4, 10000, expert_parallel_degree=8)
    cfg.model.name = "kimi_k2_7"
    return cfg
