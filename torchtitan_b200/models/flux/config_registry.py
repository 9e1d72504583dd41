"""Registered Flux training configs (parity: torchtitan/models/flux/config_registry.py)."""

from __future__ import annotations

from . import flux_configs
from .trainer import FluxTrainer


def flux_debugmodel() -> FluxTrainer.Config:
    return FluxTrainer.Config(model=flux_configs["flux-debug"](), steps=10, batch_size=2, img_size=64, txt_len=16)


def flux_dev() -> FluxTrainer.Config:
    return FluxTrainer.Config(model=flux_configs["flux-dev"](), steps=30000, batch_size=32, img_size=256, txt_len=512,
                              dtype="bfloat16")


def flux_schnell() -> FluxTrainer.Config:
    return FluxTrainer.Config(model=flux_configs["flux-schnell"](), steps=30000, batch_size=32, img_size=256, txt_len=256,
                              dtype="bfloat16")
