"""Reinforcement-learning post-training pieces (parity: torchtitan/experiments/rl): per-token
log-probabilities on folded tokens, GRPO / DAPO policy losses, group-relative advantages, a
sampling generator that runs the trainer's own model, and a rollout buffer."""

from .generator import SamplingGenerator
from .losses import dapo_loss, group_advantages, grpo_loss, token_logprobs
from .rollout import Rollout, RolloutBuffer

__all__ = ["token_logprobs", "grpo_loss", "dapo_loss", "group_advantages", "SamplingGenerator", "Rollout", "RolloutBuffer"]
