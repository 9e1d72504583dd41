"""Records that travel between the RL loops: generator -> rollout -> sample builder -> batcher -> trainer.

``Completion`` is what a generator returns for one prompt.  A ``Rollout`` is an ordered list of ``RolloutTurn``
(prompt tokens, sampled completion and its behaviour log-probabilities, the environment's reply) with a terminal
``RolloutStatus``; siblings sampled from the same prompt form a ``RolloutGroup`` (the unit of advantage
centring).  ``TrainingSample`` is a packed token sequence with a loss mask; a ``TrainingBatch`` holds the
``[microbatch][dp rank]`` grid of flat ``TrainingMicrobatch`` tensors of one optimizer step.

Parity: torchtitan/experiments/rl/types.py:15-161, rollout/types.py:29-172.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any

import torch

from .metrics import Metric

__all__ = ["Message", "RolloutTurnID", "Completion", "RolloutStatus", "RolloutTurn", "Rollout", "RolloutGroup",
           "TrainingSample", "TrainingSampleGroup", "TrainingMicrobatch", "TrainingBatch", "OptimStepOutput"]

Message = dict[str, Any]   # {"role": "system" | "user" | "assistant" | "tool", "content": str, ["tool_calls": [...]]}


@dataclass(frozen=True, kw_only=True, slots=True)
class RolloutTurnID:
    """``group`` is unique per prompt group (also the session key of sticky routing), ``rollout`` the sibling index,
    ``turn`` the turn index (for a training sample: the turn at which the sample starts)."""
    group_id: int
    rollout_id: int
    turn_id: int = 0

    def to_string(self, *, include_turn: bool = True) -> str:
        base = f"group={self.group_id}/rollout={self.rollout_id}"
        return f"{base}/turn={self.turn_id}" if include_turn else base


@dataclass(kw_only=True, slots=True)
class Completion:
    request_id: str
    token_ids: list[int]
    token_logprobs: list[float]
    finish_reason: str | None = None           # "stop" | "length" | "abort"
    min_policy_version: int = 0                # a weight swap in the middle of a decode gives min < max
    max_policy_version: int = 0
    metrics: list[Metric] = field(default_factory=list)


class RolloutStatus(str, Enum):
    ONGOING = "ongoing"
    COMPLETED = "completed"
    TRUNCATED_LENGTH = "truncated_length"
    TRUNCATED_PROMPT_TOO_LONG = "truncated_prompt_too_long"
    TRUNCATED_MAX_TURNS = "truncated_max_turns"
    ERROR_PARSE = "error_parse"
    ERROR_TIMEOUT = "error_timeout"
    ERROR_ABORT = "error_abort"
    ERROR = "error"

    def is_truncated(self) -> bool:
        return self.value.startswith("truncated")

    def is_error(self) -> bool:
        return self.value.startswith("error")

    def is_terminal(self) -> bool:
        return self is not RolloutStatus.ONGOING


@dataclass(kw_only=True, slots=True)
class RolloutTurn:
    """One generator call and the environment's answer to it."""
    rollout_id: RolloutTurnID
    # token space (what training needs)
    prompt_token_ids: list[int]                 # the whole conversation up to this turn
    completion_token_ids: list[int]
    completion_logprobs: list[float]            # behaviour policy, one per completion token
    min_policy_version: int | None = None       # None: nothing was generated
    max_policy_version: int | None = None
    # message space (what rubrics and the recorder read)
    prompt_messages: list[Message] = field(default_factory=list)
    completion_message: Message | None = None   # the environment's parse of the completion
    env_messages: list[Message] = field(default_factory=list)
    env_rewards: dict[str, float] = field(default_factory=dict)
    metrics: list[Metric] = field(default_factory=list)


@dataclass(kw_only=True, slots=True)
class Rollout:
    group_id: int
    rollout_id: int                             # sibling index inside the group
    status: RolloutStatus
    turns: list[RolloutTurn] = field(default_factory=list)
    reward: float | None = None                 # filled by the rubric
    reward_breakdown: dict[str, float] = field(default_factory=dict)
    advantage: float | None = None              # filled by the advantage estimator

    @property
    def num_completion_tokens(self) -> int:
        return sum(len(t.completion_token_ids) for t in self.turns)


@dataclass(kw_only=True, slots=True)
class RolloutGroup:
    group_id: int
    rollouts: list[Rollout]                     # empty when generation of the group failed
    metrics: list[Metric] = field(default_factory=list)


@dataclass(kw_only=True, slots=True)
class TrainingSample:
    """Packed ``prompt + completion (+ env reply + completion ...)``.  ``loss_mask`` is True on completion tokens;
    ``logprobs`` and ``advantage`` are zero elsewhere.  All four lists have the same length."""
    rollout_id: RolloutTurnID                   # turn_id: the turn at which this sample starts
    token_ids: list[int]
    loss_mask: list[bool]
    logprobs: list[float]
    advantage: list[float]
    min_policy_version: int
    max_policy_version: int

    def __len__(self) -> int:
        return len(self.token_ids)


@dataclass(frozen=True, slots=True)
class TrainingSampleGroup:
    group_id: int
    training_samples: list[TrainingSample]
    metrics: list[Metric]


@dataclass(kw_only=True, slots=True)
class TrainingMicrobatch:
    """Flat ``[T]`` tensors; a sample of N raw tokens contributes ``token_ids = raw[:-1]`` and ``labels = raw[1:]``
    (the pre-training convention), positions restart at 0 at every sample."""
    token_ids: torch.Tensor
    labels: torch.Tensor
    positions: torch.Tensor
    generator_logprobs: torch.Tensor
    loss_mask: torch.Tensor
    advantages: torch.Tensor


@dataclass(frozen=True, slots=True)
class TrainingBatch:
    microbatches: list[list[TrainingMicrobatch]]   # [num_microbatches][dp_degree]
    num_global_valid_tokens: int
    metrics: list[Metric]
    min_policy_versions: list[int]


@dataclass(frozen=True, slots=True)
class OptimStepOutput:
    policy_version: int
    metrics: dict[str, float]
