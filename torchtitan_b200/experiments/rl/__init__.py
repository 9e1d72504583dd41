"""Reinforcement-learning post-training (parity: torchtitan/experiments/rl): per-token log-probabilities on
folded tokens, GRPO / DAPO policy losses, group-relative advantages, generators that run the trainer's own model
(prefix recomputation or key/value cache), weight push to a generator's copy, a rollout buffer with staleness
eviction, the controller loop and a batch-invariant execution mode."""

from .batch_invariance import batch_invariant, enable_batch_invariant_mode
from .controller import RLConfig, RLController
from .generator import CachedGenerator, SamplingGenerator, WeightSync
from .losses import dapo_loss, group_advantages, grpo_loss, token_logprobs
from .rollout import Rollout, RolloutBuffer

__all__ = ["token_logprobs", "grpo_loss", "dapo_loss", "group_advantages", "SamplingGenerator", "CachedGenerator",
           "WeightSync", "Rollout", "RolloutBuffer", "RLConfig", "RLController", "batch_invariant",
           "enable_batch_invariant_mode"]
