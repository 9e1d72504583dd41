"""Reinforcement-learning post-training (parity: torchtitan/experiments/rl).

Two levels.  The synchronous ``RLController`` (collect -> score -> one policy step -> weight push) with the
single-sequence generators is the small loop of the unit tests.  The asynchronous stack is the production shape:
``GenerationEngine`` (continuous batching with per-sequence key/value caches on the trainer's own model code),
request routing over engine replicas, environments in message and token space, rubrics and advantage estimators,
the work buffer that bounds staleness, the packer that turns scored multi-turn rollouts into microbatch grids,
``PolicyTrainer`` and ``AsyncController``, which runs generation and training concurrently and overlaps the weight
transfer with the next step.  ``examples/`` holds two complete tasks and ``train.py`` the entry point.
"""

from . import metrics
from .async_controller import AsyncController, AsyncLoopConfig, ValidationConfig, WeightSyncManager
from .batch_invariance import batch_invariant, enable_batch_invariant_mode
from .batching import BatchConfig, Batcher, TrainingSampleBuilder
from .controller import RLConfig, RLController
from .engine import DataParallelEngine, GenerationEngine, SamplingConfig
from .environment import MessageEnv, MessageEnvInit, MessageEnvStep, TokenEnv, TokenEnvOutput
from .generator import CachedGenerator, SamplingGenerator, WeightSync
from .losses import PolicyLoss, dapo_loss, group_advantages, grpo_loss, token_logprobs
from .policy_trainer import PolicyTrainer
from .recorder import KeepExtremeRewardsFilter, RolloutSampleRecorder
from .renderer import ChatRenderer
from .rollout import RolloutBuffer, SampledResponse
from .rollouter import AdvantageEstimator, RewardFn, Rollouter, Rubric, RubricOutput
from .routing import (InterGeneratorRouter, IntraGeneratorRouter, LeastLoadedRoutingStrategy, RoundRobinRoutingStrategy,
                      RoutingContext, StickySessionRoutingStrategy)
from .records import (Completion, Rollout, RolloutGroup, RolloutStatus, RolloutTurn, RolloutTurnID, TrainingBatch,
                    TrainingMicrobatch, TrainingSample, TrainingSampleGroup)
from .work_buffer import RolloutGroupWork, RolloutGroupWorkBuffer

__all__ = [
    "token_logprobs", "grpo_loss", "dapo_loss", "group_advantages", "PolicyLoss", "SamplingGenerator", "CachedGenerator",
    "WeightSync", "SampledResponse", "RolloutBuffer", "RLConfig", "RLController", "batch_invariant",
    "enable_batch_invariant_mode", "metrics", "GenerationEngine", "DataParallelEngine", "SamplingConfig", "ChatRenderer", "MessageEnv",
    "MessageEnvInit", "MessageEnvStep", "TokenEnv", "TokenEnvOutput", "RewardFn", "Rubric", "RubricOutput",
    "AdvantageEstimator", "Rollouter", "TrainingSampleBuilder", "BatchConfig", "Batcher", "RolloutGroupWork",
    "RolloutGroupWorkBuffer", "RoutingContext", "RoundRobinRoutingStrategy", "LeastLoadedRoutingStrategy",
    "StickySessionRoutingStrategy", "IntraGeneratorRouter", "InterGeneratorRouter", "PolicyTrainer", "AsyncLoopConfig",
    "ValidationConfig", "WeightSyncManager", "AsyncController", "KeepExtremeRewardsFilter", "RolloutSampleRecorder",
    "Completion", "Rollout", "RolloutGroup", "RolloutStatus", "RolloutTurn", "RolloutTurnID", "TrainingBatch",
    "TrainingMicrobatch", "TrainingSample", "TrainingSampleGroup",
]
