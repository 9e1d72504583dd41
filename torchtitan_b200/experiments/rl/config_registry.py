"""Registered RL jobs (``python -m torchtitan_b200.experiments.rl.train --module rl --config <name>``).

Parity: torchtitan/experiments/rl/examples/alphabet_sort/config_registry.py:64-1063 (GRPO on Qwen3 0.6B ... and
its batch-invariant variants), examples/dapo_math/config_registry.py:42-160 (DAPO on Qwen3 4B, 8k / 32k tokens).
"""

from __future__ import annotations

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.data import BaseDataLoader
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ModelSelectConfig, TrainingConfig
from torchtitan_b200.trainer import Trainer

from .async_controller import AsyncController, AsyncLoopConfig, ValidationConfig
from .batching import BatchConfig, Batcher, TrainingSampleBuilder
from .engine import GenerationEngine, SamplingConfig
from .environment import TokenEnv
from .examples.alphabet_sort import AlphabetSortDataset, AlphabetSortEnv, RewardAlphabetSort
from .examples.math_answer import MathDataset, MathEnv, RewardMathAnswer
from .job import RLJob
from .rollouter import AdvantageEstimator, Rollouter, Rubric


def _trainer(name: str, flavor: str, *, lr: float, assets: str, steps: int) -> Trainer.Config:
    return Trainer.Config(
        model=ModelSelectConfig(name=name, flavor=flavor, converters=["lm_head_cast"]),
        hf_assets_path=assets,
        metrics=MetricsProcessor.Config(log_freq=1),
        dataloader=BaseDataLoader.Config(dataset="synthetic"),
        optimizer=OptimizersContainer.Config(lr=lr, weight_decay=0.0),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2, decay_ratio=None),
        training=TrainingConfig(steps=steps, max_norm=1.0),
        checkpoint=CheckpointManager.Config(enable=False))


def _alphabet_sort(seed_train: int, seed_val: int, max_turns: int) -> Rollouter.Config:
    return Rollouter.Config(
        train_dataset=AlphabetSortDataset.Config(seed=seed_train, max_turns=max_turns),
        validation_dataset=AlphabetSortDataset.Config(seed=seed_val, max_turns=max_turns),
        rubric=Rubric.Config(reward_fns=[RewardAlphabetSort.Config()], truncation_reward=0.0, error_reward=0.0),
        message_env=AlphabetSortEnv.Config(),
        token_env=TokenEnv.Config(max_num_turns=max_turns))


def rl_grpo_debug_alphabet_sort() -> RLJob.Config:
    """Debug model, byte tokenizer, a handful of steps: the smoke configuration of the RL stack (CPU or one GPU)."""
    return RLJob.Config(
        trainer=_trainer("llama3", "debugmodel", lr=1e-3, assets="", steps=4),
        byte_tokenizer=True,
        controller=AsyncController.Config(
            rollouter=_alphabet_sort(0, 99, max_turns=2),
            async_loop=AsyncLoopConfig(num_training_steps=4, num_prompts_per_train_step=2, num_samples_per_prompt=4,
                                       target_offpolicy_steps=1, batcher=Batcher.Config(batch=BatchConfig(local_batch_size=2, seq_len=1024)),
                                       validation=ValidationConfig(num_samples=2),
                                       # a random-init model never answers in the asked format: every reward is 0
                                       training_sample_builder=TrainingSampleBuilder.Config(drop_zero_std_reward_groups=False)),
            sampling=SamplingConfig(max_tokens=24)),
        generator=GenerationEngine.Config(max_num_seqs=16))


def rl_grpo_qwen3_0_6b_alphabet_sort() -> RLJob.Config:
    """GRPO on Qwen3 0.6B, multi-turn alphabet sort; the generator decodes on the training weights."""
    return RLJob.Config(
        trainer=_trainer("qwen3", "0.6B", lr=1e-6, assets="./assets/hf/Qwen3-0.6B", steps=100),
        controller=AsyncController.Config(
            rollouter=_alphabet_sort(1337420, 99, max_turns=3),
            async_loop=AsyncLoopConfig(num_training_steps=100, num_prompts_per_train_step=8, num_samples_per_prompt=8,
                                       target_offpolicy_steps=1, batcher=Batcher.Config(batch=BatchConfig(local_batch_size=4, seq_len=4096)),
                                       validation=ValidationConfig(num_samples=20)),
            sampling=SamplingConfig(temperature=1.0, max_tokens=512)),
        generator=GenerationEngine.Config(max_num_seqs=64, max_batched_tokens=16384))


def rl_grpo_qwen3_0_6b_alphabet_sort_batch_invariant() -> RLJob.Config:
    """As above with batch-invariant kernels, deterministic mode and per-sample padding, so that the trainer's
    log-probabilities of a sample do not depend on what it is packed with."""
    cfg = rl_grpo_qwen3_0_6b_alphabet_sort()
    cfg.trainer.debug.batch_invariant = True
    cfg.trainer.debug.deterministic = True
    cfg.controller.async_loop.batcher.per_sample_pad_multiple = 128
    return cfg


def rl_grpo_qwen3_0_6b_async_two_generators() -> RLJob.Config:
    """Trainer on GPU 0, two generator replicas with their own weights on GPUs 1 and 2, three steps off-policy."""
    cfg = rl_grpo_qwen3_0_6b_alphabet_sort()
    cfg.share_weights, cfg.num_generators = False, 2
    cfg.generator_devices = ["cuda:1", "cuda:2"]
    cfg.controller.async_loop.target_offpolicy_steps = 3
    return cfg


def rl_dapo_qwen3_4b_math_8k() -> RLJob.Config:
    """DAPO (clip-higher, zero-variance groups dropped, std-normalised advantages) on Qwen3 4B with verifiable
    math answers and 8k-token rows."""
    return RLJob.Config(
        trainer=_trainer("qwen3", "4B", lr=1e-6, assets="./assets/hf/Qwen3-4B", steps=200),
        ratio_clip_low=0.2, ratio_clip_high=0.28,
        controller=AsyncController.Config(
            rollouter=Rollouter.Config(
                train_dataset=MathDataset.Config(path="./assets/datasets/dapo_math_17k.jsonl", seed=0),
                validation_dataset=MathDataset.Config(path="./assets/datasets/aime_2025.jsonl", seed=0, num_samples=30),
                rubric=Rubric.Config(reward_fns=[RewardMathAnswer.Config()], truncation_reward=0.0),
                message_env=MathEnv.Config(),
                advantage=AdvantageEstimator.Config(should_std_normalize=True)),
            async_loop=AsyncLoopConfig(num_training_steps=200, num_prompts_per_train_step=32, num_samples_per_prompt=16,
                                       target_offpolicy_steps=1, batcher=Batcher.Config(batch=BatchConfig(local_batch_size=1, seq_len=8192)),
                                       validation=ValidationConfig(num_samples=30)),
            sampling=SamplingConfig(temperature=1.0, top_p=1.0, max_tokens=7168)),
        generator=GenerationEngine.Config(max_num_seqs=128, max_batched_tokens=32768))
