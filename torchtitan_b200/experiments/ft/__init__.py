"""Fault-tolerant replicated training (parity: torchtitan/experiments/torchft): replica-group
membership with heartbeats and a per-step quorum, gradient averaging among the live replicas,
commit / rollback of a step, and the semi-synchronous LocalSGD / DiLoCo algorithms."""

from .manager import FTManager, QuorumResult
from .semi_sync import DiLoCo, LocalSGD

__all__ = ["FTManager", "QuorumResult", "LocalSGD", "DiLoCo"]
