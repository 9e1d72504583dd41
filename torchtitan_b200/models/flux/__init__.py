"""Flux diffusion transformers (parity: torchtitan/models/flux/__init__.py): flux-dev, flux-schnell, flux-debug."""

from __future__ import annotations

from torchtitan_b200.models.spec import ModelSpec

from .model import FluxModel

__all__ = ["flux_configs", "model_registry", "FluxModel"]

flux_configs = {
    "flux-debug": lambda: FluxModel.Config(in_channels=64, out_channels=64, vec_in_dim=64, context_in_dim=96, hidden_size=128,
                                           num_heads=4, depth=2, depth_single_blocks=2, axes_dim=(8, 12, 12)),
    "flux-dev": lambda: FluxModel.Config(),
    "flux-schnell": lambda: FluxModel.Config(),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in flux_configs:
        raise ValueError(f"unknown flux flavor '{flavor}' (have {sorted(flux_configs)})")
    return ModelSpec(name="flux", flavor=flavor, model=flux_configs[flavor]())
