"""Registered Qwen3 training configs (parity: torchtitan/models/qwen3/config_registry.py:37-462)."""

from __future__ import annotations

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.data import BaseDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer, ParamGroupConfig
from torchtitan_b200.config import ActivationCheckpointConfig, ModelSelectConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.trainer import Trainer


def _debug(flavor: str) -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="qwen3", flavor=flavor),
        metrics=MetricsProcessor.Config(log_freq=1),
        dataloader=BaseDataLoader.Config(dataset="synthetic"),
        optimizer=OptimizersContainer.Config(lr=3e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=8 * 2048, max_context_length=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective"),
    )


def qwen3_debugmodel() -> Trainer.Config:
    return _debug("debugmodel")


def qwen3_moe_debug() -> Trainer.Config:
    return _debug("debugmodel_moe")


def qwen3_moe_debug_param_groups() -> Trainer.Config:
    cfg = _debug("debugmodel_moe")
    cfg.optimizer.param_groups = [
        ParamGroupConfig(pattern=r"moe\.routed_experts", optimizer_name="AdamW", optimizer_kwargs={"lr": 1e-4}),
        ParamGroupConfig(pattern=r"norm", optimizer_name="AdamW", optimizer_kwargs={"weight_decay": 0.0}),
    ]
    return cfg


def _full(flavor: str, tokens: int, ctx: int, lr: float, ac: str = "selective", **par) -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="qwen3", flavor=flavor),
        hf_assets_path=f"./assets/hf/Qwen3-{flavor}",
        dataloader=BaseDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=lr),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=600),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=tokens, max_context_length=ctx, steps=3000),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, **par),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode=ac),
    )


def qwen3_0_6b() -> Trainer.Config:
    return _full("0.6B", 4 * 4096, 4096, 3e-4)


def qwen3_1_7b() -> Trainer.Config:
    return _full("1.7B", 4 * 4096, 4096, 8e-4)


def qwen3_8b() -> Trainer.Config:
    return _full("8B", 4096, 4096, 3e-4)


def qwen3_14b() -> Trainer.Config:
    return _full("14B", 4 * 4096, 4096, 8e-4, ac="full", tensor_parallel_degree=4)


def qwen3_32b() -> Trainer.Config:
    return _full("32B", 2 * 4096, 4096, 8e-4, ac="full", tensor_parallel_degree=8)


def qwen3_30b_a3b() -> Trainer.Config:
    return _full("30B-A3B", 8192, 4096, 8e-4, ac="full")


def qwen3_30b_a3b_ep8() -> Trainer.Config:
    """Expert parallel over 8 GPUs with non-expert parameters sharded over the same ranks."""
    return _full("30B-A3B", 8192, 4096, 8e-4, ac="selective", expert_parallel_degree=8)


def qwen3_235b_a22b() -> Trainer.Config:
    return _full("235B-A22B", 4 * 4096, 4096, 8e-4, ac="full", expert_parallel_degree=8, tensor_parallel_degree=1)
