"""Registered Muse Glimmer training configs (parity: torchtitan/models/muse_glimmer/config_registry.py)."""

from __future__ import annotations

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.data import BaseDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, ModelSelectConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.trainer import Trainer


def muse_glimmer_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="muse_glimmer", flavor="debugmodel"),
        metrics=MetricsProcessor.Config(log_freq=1),
        dataloader=BaseDataLoader.Config(dataset="synthetic"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=8 * 2048, max_context_length=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective"),
    )


def muse_glimmer_debugmodel_mm() -> Trainer.Config:
    cfg = muse_glimmer_debugmodel()
    cfg.model.flavor = "debugmodel_mm"
    cfg.dataloader.dataset = "synthetic_mm"
    return cfg


def muse_glimmer_30b() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="muse_glimmer", flavor="30B"),
        dataloader=BaseDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=3e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2000),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=16384, max_context_length=16384, steps=10000),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, tensor_parallel_degree=2),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def muse_glimmer_30b_mm() -> Trainer.Config:
    cfg = muse_glimmer_30b()
    cfg.model.flavor = "30B_mm"
    cfg.dataloader.dataset = "mm_jsonl"
    return cfg
