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


def qwen3_moe_tiny() -> Trainer.Config:
    """Two layers of eight experts at width 64: the mixture-of-experts model of the CPU multi-rank tests."""
    return _debug("debugmodel_moe_tiny")


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


def qwen3_debugmodel_nvfp4() -> Trainer.Config:
    cfg = qwen3_debugmodel()
    cfg.model.converters = ["nvfp4"]
    return cfg


def qwen3_debugmodel_first_85_pct_layers_nvfp4() -> Trainer.Config:
    cfg = qwen3_debugmodel()
    cfg.model.converters = ["nvfp4:tail=0.15"]
    return cfg


def qwen3_8b_first_85_pct_layers_nvfp4() -> Trainer.Config:
    cfg = qwen3_8b()
    cfg.model.converters = ["nvfp4:tail=0.15"]
    return cfg


def qwen3_moe_nvlink_ep() -> Trainer.Config:
    """MoE debug model with expert parallelism over NVLink peer stores (no all-to-all, no host sync)."""
    cfg = qwen3_moe_debug()
    cfg.parallelism.expert_parallel_degree = 2
    cfg.parallelism.ep_comm = "nvlink"
    return cfg


def sft_qwen3_8b_math() -> Trainer.Config:
    """Single-turn supervised fine-tuning (prompt tokens masked) of the 8B model on a question / answer set."""
    from torchtitan_b200.components.data import BaseDataLoader

    cfg = qwen3_8b()
    cfg.dataloader = BaseDataLoader.Config(dataset="sft_test", packing="first_fit")
    cfg.optimizer.lr = 1e-5
    cfg.training.steps = 500
    return cfg
