"""Rewards, advantages and the rollout driver.

``RewardFn`` scores one rollout; a ``Rubric`` combines several with normalised weights and can short-circuit
truncated / errored rollouts to fixed rewards.  ``AdvantageEstimator`` centres rewards inside a prompt group
(``(r - mean) / (std + eps)`` for GRPO, mean baseline only for Dr.GRPO).  ``Rollouter`` owns the datasets, builds
``group_size`` sibling environments per dataset sample, drives each against a ``generate_fn`` (any awaitable
``prompt tokens -> Completion``: an engine, a router over several engines) until its environment is terminal, then
scores the group and fills the advantages.

Parity: torchtitan/experiments/rl/rubrics/rubric.py:18-177, rollout/advantage.py:22-46, rollout/rollouter.py:36-314.
"""

from __future__ import annotations

import abc
import asyncio
import dataclasses
import statistics
from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from .environment import MessageEnv, TokenEnv
from .records import Completion, Rollout, RolloutGroup, RolloutStatus, RolloutTurn, RolloutTurnID

__all__ = ["RewardFn", "RubricOutput", "Rubric", "AdvantageEstimator", "Rollouter", "GenerateFn"]

GenerateFn = Callable[..., Awaitable[Completion | None]]
"""``await generate_fn(prompt_token_ids, request_id=..., routing_session_id=..., sampling_config=...)``."""


class RewardFn(Configurable, abc.ABC):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        weight: float = 1.0

    def __init__(self, config: "RewardFn.Config | None" = None, **_):
        self.config = config or type(self).Config()
        self.weight = self.config.weight

    @abc.abstractmethod
    async def __call__(self, rollout: Rollout, env_input: Any) -> float: ...


@dataclass(frozen=True, kw_only=True, slots=True)
class RubricOutput:
    reward: float
    reward_breakdown: dict[str, float] = field(default_factory=dict)   # unweighted, by reward-function class name


class Rubric(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        reward_fns: list[RewardFn.Config] = field(default_factory=list)
        truncation_reward: float | None = None
        """Fixed reward of a truncated rollout (the reward functions are skipped); None: they run as usual."""
        error_reward: float | None = None

    def __init__(self, config: Config, **_):
        self.config = config
        self.fns = [c.build() for c in config.reward_fns]
        if not self.fns:
            raise ValueError("a rubric needs at least one reward function")
        names = [type(f).__name__ for f in self.fns]
        if len(set(names)) != len(names):
            raise ValueError(f"reward function names must be unique, got {names}")
        self._wsum = sum(f.weight for f in self.fns)
        if self._wsum <= 0:
            raise ValueError(f"reward weights must sum to a positive value, got {self._wsum}")

    async def score(self, rollout: Rollout, env_input: Any) -> RubricOutput:
        c = self.config
        if c.truncation_reward is not None and rollout.status.is_truncated():
            return RubricOutput(reward=c.truncation_reward, reward_breakdown={"truncated": c.truncation_reward})
        if c.error_reward is not None and rollout.status.is_error():
            return RubricOutput(reward=c.error_reward, reward_breakdown={"errored": c.error_reward})
        raw = await asyncio.gather(*(f(rollout, env_input) for f in self.fns))
        parts = {type(f).__name__: float(r) for f, r in zip(self.fns, raw)}
        return RubricOutput(reward=sum(f.weight / self._wsum * float(r) for f, r in zip(self.fns, raw)),
                            reward_breakdown=parts)

    async def score_group(self, rollouts: list[Rollout], env_input: Any) -> list[RubricOutput]:
        """Override for rewards that compare siblings (pairwise judges, diversity, rank normalisation)."""
        return list(await asyncio.gather(*(self.score(r, env_input) for r in rollouts)))


class AdvantageEstimator(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        should_std_normalize: bool = False
        """Divide by the group's reward std (GRPO); off: mean baseline only (Dr.GRPO)."""

    def __init__(self, config: Config | None = None, **_):
        self.config = config or AdvantageEstimator.Config()

    def __call__(self, group: RolloutGroup) -> list[float]:
        r = [float(x.reward) for x in group.rollouts]
        mu = sum(r) / len(r)
        denom = statistics.pstdev(r) + 1e-6 if self.config.should_std_normalize else 1.0
        return [(x - mu) / denom for x in r]


class Rollouter(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        train_dataset: Configurable.Config
        """Builds an iterator whose ``next()`` is one environment input."""
        validation_dataset: Configurable.Config
        rubric: Rubric.Config
        message_env: MessageEnv.Config
        token_env: TokenEnv.Config = field(default_factory=TokenEnv.Config)
        advantage: AdvantageEstimator.Config = field(default_factory=AdvantageEstimator.Config)

    def __init__(self, config: Config, **_):
        self.config = config
        self._train, self._val = config.train_dataset.build(), config.validation_dataset.build()
        self.rubric: Rubric = config.rubric.build()
        self.advantage_estimator = config.advantage.build()

    def get_training_sample(self) -> Any:
        return next(self._train)

    def get_validation_sample(self) -> Any:
        return next(self._val)

    def dataset_state(self) -> dict:
        return {k: d.state_dict() for k, d in (("train", self._train), ("validation", self._val)) if hasattr(d, "state_dict")}

    def load_dataset_state(self, state: dict) -> None:
        for k, d in (("train", self._train), ("validation", self._val)):
            if k in state and hasattr(d, "load_state_dict"):
                d.load_state_dict(state[k])

    def make_env_group(self, *, sample: Any, group_size: int, renderer) -> list[TokenEnv]:
        return [self.config.token_env.build(message_env=self.config.message_env.build(env_input=sample), renderer=renderer)
                for _ in range(group_size)]

    async def score_group(self, rollouts: list[Rollout], env_input: Any) -> list[RubricOutput]:
        return await self.rubric.score_group(rollouts, env_input)

    async def run_group_rollouts(self, *, generate_fn: GenerateFn, sample: Any, group_id: int, group_size: int,
                                 sampling, renderer) -> RolloutGroup:
        envs = self.make_env_group(sample=sample, group_size=group_size, renderer=renderer)

        def seeded(i):     # siblings must not share a sampling seed
            if sampling is None or getattr(sampling, "seed", None) is None:
                return sampling
            return dataclasses.replace(sampling, seed=sampling.seed + i)

        try:
            rollouts = list(await asyncio.gather(*(
                self._run_single_rollout(generate_fn=generate_fn, env=env, sampling=seeded(i), group_id=group_id, rollout_id=i)
                for i, env in enumerate(envs))))
        finally:
            await asyncio.gather(*(e.close() for e in envs), return_exceptions=True)
        for r, out in zip(rollouts, await self.score_group(rollouts, sample), strict=True):
            r.reward, r.reward_breakdown = out.reward, out.reward_breakdown
        group = RolloutGroup(group_id=group_id, rollouts=rollouts)
        for r, a in zip(rollouts, self.advantage_estimator(group), strict=True):
            r.advantage = a
        return group

    async def _run_single_rollout(self, *, generate_fn: GenerateFn, env: TokenEnv, sampling, group_id: int,
                                  rollout_id: int) -> Rollout:
        turns: list[RolloutTurn] = []
        status = RolloutStatus.ERROR
        try:
            out = await env.init()
            while not out.status.is_terminal():
                tid = RolloutTurnID(group_id=group_id, rollout_id=rollout_id, turn_id=len(turns))
                completion = await generate_fn(out.next_prompt_token_ids, request_id=tid.to_string(),
                                               routing_session_id=tid.to_string(include_turn=False),
                                               sampling_config=sampling)
                if completion is None:
                    raise RuntimeError(f"{tid.to_string()}: the generator returned no completion")
                nxt = await env.step(completion)
                turns.append(RolloutTurn(
                    rollout_id=tid, prompt_token_ids=out.next_prompt_token_ids or [],
                    prompt_messages=out.next_prompt_messages or [], completion_token_ids=completion.token_ids,
                    completion_logprobs=completion.token_logprobs, completion_message=nxt.completion_message,
                    env_messages=nxt.env_messages, env_rewards=nxt.env_rewards,
                    min_policy_version=completion.min_policy_version, max_policy_version=completion.max_policy_version,
                    metrics=completion.metrics))
                out = nxt
            status = out.status
        except Exception:
            logger.exception(f"rollout group={group_id}/rollout={rollout_id} failed after {len(turns)} turn(s)")
            status = RolloutStatus.ERROR
        return Rollout(group_id=group_id, rollout_id=rollout_id, status=status, turns=turns)
