"""Registered fault-tolerant jobs (``--module ft --config llama3_ft_debugmodel``; one launch per replica group, each
with its own ``--fault_tolerance.replica_id``).

Parity: torchtitan/experiments/torchft/llama3/config_registry.py:25-75.
"""

from __future__ import annotations

import dataclasses

from torchtitan_b200.models.llama3.config_registry import llama3_debugmodel

from .trainer import FaultToleranceConfig, FaultTolerantTrainer


def _as_ft(base, **ft) -> FaultTolerantTrainer.Config:
    shared = {f.name: getattr(base, f.name) for f in dataclasses.fields(base) if not f.name.startswith("_")}
    return FaultTolerantTrainer.Config(**shared, fault_tolerance=FaultToleranceConfig(enable=True, **ft))


def llama3_ft_debugmodel() -> FaultTolerantTrainer.Config:
    """Two replica groups of the debug model averaging gradients every step."""
    return _as_ft(llama3_debugmodel(), group_size=2, min_replica_size=1)


def llama3_ft_debugmodel_diloco() -> FaultTolerantTrainer.Config:
    """DiLoCo: local AdamW steps, outer Nesterov step on the averaged pseudo-gradients every 5 steps, two fragments."""
    return _as_ft(llama3_debugmodel(), group_size=2, semi_sync_method="diloco", sync_steps=5, num_fragments=2)
