"""Registered Llama-3 training configs (``--module llama3 --config <name>``).

Parity: torchtitan/models/llama3/config_registry.py:38-411 (debug model: 10 steps,
lr 8e-4, warmup 2, decay ratio 0.8; 8B: lr 3e-4, local batch 1 x 8192, selective AC;
70B / 405B: full AC with tensor (and pipeline) parallelism).
"""

from __future__ import annotations

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.data import BaseDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, ModelSelectConfig, ParallelismConfig, TrainingConfig
from torchtitan_b200.trainer import Trainer


def llama3_debugmodel() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="llama3", flavor="debugmodel"),
        metrics=MetricsProcessor.Config(log_freq=1),
        dataloader=BaseDataLoader.Config(dataset="synthetic"),
        optimizer=OptimizersContainer.Config(lr=8e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=0.8, decay_type="linear", min_lr_factor=0.0),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=8 * 2048, max_context_length=2048, steps=10),
        checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective"),
    )


def llama3_debugmodel_hd128() -> Trainer.Config:
    """Debug model whose attention has head dimension 128 (runs the flash-attention kernels)."""
    cfg = llama3_debugmodel()
    cfg.model.flavor = "debugmodel_hd128"
    return cfg


def llama3_debugmodel_c4() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.dataloader = BaseDataLoader.Config(dataset="c4_test")
    return cfg


def llama3_debugmodel_mxfp8() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model.converters = ["mxfp8"]
    return cfg


def llama3_debugmodel_float8() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model.converters = ["float8"]
    return cfg


def llama3_debugmodel_float8_emulate_lora() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model.converters = ["float8:emulate", "lora"]
    return cfg


def llama3_8b() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="llama3", flavor="8B"),
        hf_assets_path="./assets/hf/Llama-3.1-8B",
        dataloader=BaseDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=3e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=200),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=8192, max_context_length=8192, steps=1000),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="selective", selective_ac_option="op"),
    )


def llama3_8b_mxfp8() -> Trainer.Config:
    cfg = llama3_8b()
    cfg.model.converters = ["mxfp8"]
    return cfg


def llama3_70b() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="llama3", flavor="70B"),
        hf_assets_path="./assets/hf/Llama-3.1-70B",
        dataloader=BaseDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=1.5e-4),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=200),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=8 * 8192, max_context_length=8192, steps=1000),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, tensor_parallel_degree=8),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def llama3_405b() -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name="llama3", flavor="405B"),
        hf_assets_path="./assets/hf/Llama-3.1-405B",
        dataloader=BaseDataLoader.Config(dataset="c4"),
        optimizer=OptimizersContainer.Config(lr=8e-5),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=600),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=2 * 8192, max_context_length=8192, steps=3000),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, tensor_parallel_degree=8,
                                      pipeline_parallel_degree=1),
        checkpoint=CheckpointManager.Config(interval=500),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
    )


def sft_debugmodel() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.dataloader = BaseDataLoader.Config(dataset="sft_test")
    return cfg


def llama3_debugmodel_varlen_attn() -> Trainer.Config:
    """Packed documents of varying length through the native flash kernel (document starts from positions)."""
    cfg = llama3_debugmodel()
    cfg.dataloader = BaseDataLoader.Config(dataset="synthetic", synthetic_doc_len=512)
    return cfg


def llama3_debugmodel_dist_gemm() -> Trainer.Config:
    """Tensor + sequence parallel with the all-gather / reduce-scatter fused into the GEMM kernels."""
    cfg = llama3_debugmodel()
    cfg.parallelism.tensor_parallel_degree = 2
    cfg.parallelism.enable_sequence_parallel = True
    cfg.parallelism.tp_comm = "nvlink"
    return cfg


def llama3_debugmodel_nvfp4() -> Trainer.Config:
    cfg = llama3_debugmodel()
    cfg.model.converters = ["nvfp4"]
    return cfg


def llama3_debugmodel_first_85_pct_layers_nvfp4() -> Trainer.Config:
    """NVFP4 for the leading 85 % of the layers, the tail stays bf16."""
    cfg = llama3_debugmodel()
    cfg.model.converters = ["nvfp4:tail=0.15"]
    return cfg


def llama3_debugmodel_ce_loss() -> Trainer.Config:
    """Plain cross entropy on materialised logits instead of the chunked fused lm_head + loss."""
    cfg = llama3_debugmodel()
    cfg.loss.name = "cross_entropy"
    return cfg


def llama3_8b_first_85_pct_layers_nvfp4() -> Trainer.Config:
    cfg = llama3_8b()
    cfg.model.converters = ["nvfp4:tail=0.15"]
    return cfg
