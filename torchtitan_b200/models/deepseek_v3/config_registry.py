"""Registered DeepSeek-V3 training configs (parity: torchtitan/models/deepseek_v3/config_registry.py)."""

from __future__ import annotations

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.data import BaseDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, ModelSelectConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.trainer import Trainer


def deepseek_v3_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="deepseek_v3", flavor="debugmodel"),
        metrics=MetricsProcessor.Config(log_freq=1),
        dataloader=BaseDataLoader.Config(dataset="synthetic"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=8 * 2048, max_context_length=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective"),
    )


def deepseek_v3_debugmodel_mtp() -> Trainer.Config:
    """Debug model with two multi-token-prediction depths."""
    cfg = deepseek_v3_debugmodel()
    cfg.model.flavor = "debugmodel_mtp"
    return cfg


def _full(flavor: str, tokens: int, ctx: int, lr: float, steps: int, **par) -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="deepseek_v3", flavor=flavor),
        hf_assets_path=f"./assets/hf/DeepSeek-V3-{flavor}",
        dataloader=BaseDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=lr),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2000, decay_ratio=0.8, decay_type="cosine", min_lr_factor=0.1),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=tokens, max_context_length=ctx, steps=steps),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, **par),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def deepseek_v3_16b() -> Trainer.Config:
    return _full("16B", 4 * 4096, 4096, 2.2e-4, 10000, expert_parallel_degree=8)


def deepseek_v3_236b() -> Trainer.Config:
    return _full("236B", 4 * 4096, 4096, 2.2e-4, 10000, expert_parallel_degree=8)


def deepseek_v3_671b() -> Trainer.Config:
    return _full("671B", 4 * 4096, 4096, 2.2e-4, 10000, expert_parallel_degree=8)


def deepseek_v3_debugmodel_mxfp8() -> Trainer.Config:
    """Block-scaled MXFP8 for the dense linears and the grouped expert GEMMs."""
    cfg = deepseek_v3_debugmodel()
    cfg.model.converters = ["mxfp8", "mxfp8_experts"]
    return cfg


def deepseek_v3_debugmodel_minimal_async_ep() -> Trainer.Config:
    """Expert parallelism with direct peer-memory row copies: no host sync, CUDA-graph capturable."""
    cfg = deepseek_v3_debugmodel()
    cfg.parallelism.expert_parallel_degree = 2
    cfg.parallelism.ep_comm = "nvlink"
    return cfg


def deepseek_v3_16b_minimal_async_ep() -> Trainer.Config:
    cfg = deepseek_v3_16b()
    cfg.parallelism.ep_comm = "nvlink"
    return cfg


def deepseek_v3_671b_float8() -> Trainer.Config:
    cfg = deepseek_v3_671b()
    cfg.model.converters = ["float8", "float8_experts"]
    return cfg
