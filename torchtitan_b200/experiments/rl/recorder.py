"""Rollouts on disk for inspection, and the metrics derived from rollouts and from the step timers.

``RolloutSampleRecorder`` appends one JSON object per selected rollout to ``<dump_dir>/rollout_samples.jsonl``
(messages, status, reward and its breakdown, advantage, policy versions per turn; token ids and log-probabilities
only on request); ``KeepExtremeRewardsFilter`` selects the ``k`` best and ``k`` worst rollouts of each group.

Parity: torchtitan/experiments/rl/rollout_recorder.py:33-147, controller_metrics.py:56-278.
"""

from __future__ import annotations

import json
import os
from collections import defaultdict
from dataclasses import dataclass, field

from torchtitan_b200.config import Configurable

from . import metrics as m
from .records import Rollout, RolloutGroup

__all__ = ["KeepExtremeRewardsFilter", "RolloutSampleRecorder", "compute_rollout_metrics", "compute_policy_age_metrics",
           "compute_perf_ratio_metrics", "combine_microbatch_metrics"]


class KeepExtremeRewardsFilter(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        k: int = 1

    def __init__(self, config: Config | None = None, **_):
        self.k = (config or KeepExtremeRewardsFilter.Config()).k

    def __call__(self, groups: list[RolloutGroup]) -> list[Rollout]:
        out: list[Rollout] = []
        for g in groups:
            ranked = sorted((r for r in g.rollouts if r.reward is not None), key=lambda r: r.reward)
            out += ranked if len(ranked) <= 2 * self.k else ranked[:self.k] + ranked[-self.k:]
        return out


class RolloutSampleRecorder(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        filter: KeepExtremeRewardsFilter.Config = field(default_factory=KeepExtremeRewardsFilter.Config)
        filename: str = "rollout_samples.jsonl"
        log_tensors: bool = False
        log_logprobs: bool = False

    def __init__(self, config: Config | None = None, *, dump_dir: str):
        self.config = config or RolloutSampleRecorder.Config()
        self._filter = self.config.filter.build()
        os.makedirs(dump_dir, exist_ok=True)
        self.path = os.path.join(dump_dir, self.config.filename)

    def record(self, *, is_validation: bool, rollout_groups: list[RolloutGroup], step: int | None = None) -> int:
        lines = []
        for r in self._filter(rollout_groups):
            lines.append(json.dumps({
                "is_validation": is_validation, "step": step, "group_id": r.group_id, "rollout_id": r.rollout_id,
                "status": r.status.value, "reward": r.reward, "reward_breakdown": r.reward_breakdown,
                "advantage": r.advantage, "turns": [self._turn(t) for t in r.turns]}, default=str) + "\n")
        with open(self.path, "a", encoding="utf-8") as f:
            f.write("".join(lines))
        return len(lines)

    def _turn(self, t) -> dict:
        d = {"turn_id": t.rollout_id.turn_id, "min_policy_version": t.min_policy_version,
             "max_policy_version": t.max_policy_version, "prompt_messages": t.prompt_messages,
             "completion_message": t.completion_message, "env_messages": t.env_messages, "env_rewards": t.env_rewards}
        if self.config.log_tensors:
            d["prompt_token_ids"], d["completion_token_ids"] = t.prompt_token_ids, t.completion_token_ids
        if self.config.log_logprobs:
            d["completion_logprobs"] = t.completion_logprobs
        return d


def compute_rollout_metrics(prefix: str, rollouts: list[Rollout]) -> list[m.Metric]:
    """Lengths, turns, truncation rate, reward statistics and per-reward-function means, plus whatever each
    generation call measured (those keep their own keys)."""
    comp = [len(t.completion_token_ids) for r in rollouts for t in r.turns]
    prompt = [len(r.turns[0].prompt_token_ids) for r in rollouts if r.turns]
    total = [len(r.turns[-1].prompt_token_ids) + len(r.turns[-1].completion_token_ids) for r in rollouts if r.turns]
    out = [m.Metric(f"{prefix}/response_length", m.Mean.from_list(comp)),
           m.Metric(f"{prefix}/response_length", m.Std.from_list(comp)),
           m.Metric(f"{prefix}/response_length", m.Max.from_list(comp)),
           m.Metric(f"{prefix}/prompt_length", m.Mean.from_list(prompt)),
           m.Metric(f"{prefix}/prompt_length", m.Max.from_list(prompt)),
           m.Metric(f"{prefix}/total_length", m.Mean.from_list(total)),
           m.Metric(f"{prefix}/total_length", m.Max.from_list(total)),
           m.Metric(f"{prefix}/num_turns", m.Mean.from_list([len(r.turns) for r in rollouts])),
           m.Metric(f"{prefix}/num_turns", m.Max.from_list([len(r.turns) for r in rollouts])),
           m.Metric(f"{prefix}/truncation_rate", m.Mean.from_list([float(r.status.is_truncated()) for r in rollouts])),
           m.Metric(f"{prefix}/error_rate", m.Mean.from_list([float(r.status.is_error()) for r in rollouts])),
           m.Metric(f"{prefix}_reward", m.SummaryStats.from_list([r.reward for r in rollouts if r.reward is not None]))]
    parts: dict[str, list[float]] = defaultdict(list)
    for r in rollouts:
        for k, v in r.reward_breakdown.items():
            parts[k].append(float(v))
    out += [m.Metric(f"{prefix}_reward/component/{k}", m.Mean.from_list(v)) for k, v in sorted(parts.items())]
    out += [x for r in rollouts for t in r.turns for x in t.metrics]
    return out


def compute_policy_age_metrics(*, trainer_policy_version: int, min_policy_versions: list[int],
                               max_offpolicy_steps: int) -> list[m.Metric]:
    """Age (in optimizer steps) of every packed sample at the moment the trainer consumes it.  An age beyond
    the bound the buffer guarantees means the back-pressure is broken: that raises instead of training on it."""
    ages = [trainer_policy_version - v for v in min_policy_versions]
    worst = max(ages, default=0)
    if worst > max_offpolicy_steps:
        raise RuntimeError(f"stale training data admitted: policy age {worst} > bound {max_offpolicy_steps} "
                           f"(trainer at version {trainer_policy_version})")
    return [m.Metric("policy_age", m.Mean.from_list(ages)), m.Metric("policy_age_max", m.NoReduce(float(worst)))]


def compute_perf_ratio_metrics(*, num_global_valid_tokens: int, time_metrics: list[m.Metric]) -> list[m.Metric]:
    t = {x.key: x.value.total for x in time_metrics}
    step = t.get("timing/step/total")
    if not step:
        return []
    out = [m.Metric("perf/trainer/tokens_per_second_full_step", m.NoReduce(num_global_valid_tokens / step))]
    names = {"wait_for_training_batch": "batch", "blocking_trainer_push": "blocking_trainer_push",
             "blocking_generator_pull": "blocking_generator_pull"}
    for key, short in names.items():
        if f"timing/step/{key}" in t:
            out.append(m.Metric(f"perf/trainer/step_time_ratio/{short}", m.NoReduce(t[f"timing/step/{key}"] / step)))
    fb, opt = t.get("timing/step/forward_backward"), t.get("timing/step/optim")
    if fb is not None and opt is not None:
        out.append(m.Metric("perf/trainer/step_time_ratio/fwd_bwd", m.NoReduce((fb + opt) / step)))
        if fb + opt:
            out.append(m.Metric("perf/trainer/tokens_per_second_fwd_bwd", m.NoReduce(num_global_valid_tokens / (fb + opt))))
    parts = [t.get(f"timing/step/{k}") for k in (*names, "forward_backward", "optim")]
    if None not in parts:
        out.append(m.Metric("perf/trainer/step_time_ratio/unaccounted", m.NoReduce((step - sum(parts)) / step)))
    return out


def combine_microbatch_metrics(per_microbatch: list[dict[str, float]]) -> dict[str, float]:
    """The loss metrics of a microbatch are already divided by the step's global token count: sums add up, maxima
    take the max."""
    out: dict[str, float] = {}
    for d in per_microbatch:
        for k, v in d.items():
            if k not in out:
                out[k] = v
            elif k.endswith("/max"):
                out[k] = max(out[k], v)
            else:
                out[k] += v
    return out
