"""Fault-tolerant replicated training (parity: torchtitan/experiments/torchft): replica-group
membership with heartbeats and a per-step quorum, gradient averaging among the live replicas,
commit / rollback of a step, the semi-synchronous LocalSGD / DiLoCo algorithms, and the trainer / optimizer /
checkpoint wrappers that put them under the regular training loop."""

from .manager import FTManager, QuorumResult
from .semi_sync import DiLoCo, LocalSGD
from .trainer import (FaultToleranceConfig, FaultTolerantTrainer, FTCheckpointManager, FTOptimizersContainer,
                      fragment_llm)

__all__ = ["FTManager", "QuorumResult", "LocalSGD", "DiLoCo", "FaultToleranceConfig", "FaultTolerantTrainer",
           "FTCheckpointManager", "FTOptimizersContainer", "fragment_llm"]
