"""From scored rollout groups to the tensors of one optimizer step.

``TrainingSampleBuilder`` filters a group (no completion at all -> untrainable; all rewards equal -> no signal,
dropped by default) and packs each rollout into training samples: turns whose prompt extends the previous
``prompt + completion`` token for token are merged into ONE sample (prompts and environment replies masked out,
completions trained); where that prefix breaks (history compacted, reasoning stripped, re-tokenisation) a new
sample starts.  ``Batcher`` collects groups until ``num_prompts_per_train_step`` trainable ones are present, packs
their samples next-fit into rows of ``seq_len`` tokens, pads the row count to a multiple of ``local_batch_size x
dp_degree`` and deals the rows round-robin into a ``[microbatch][dp rank]`` grid of flat microbatches.

Parity: torchtitan/experiments/rl/components/training_sample_builder.py:25-244, components/batcher.py:46-419.
"""

from __future__ import annotations

import dataclasses
import math
import statistics
from dataclasses import dataclass, field

import torch

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from . import metrics as m
from .records import (Rollout, RolloutGroup, RolloutTurnID, TrainingBatch, TrainingMicrobatch, TrainingSample,
                    TrainingSampleGroup)

__all__ = ["TrainingSampleBuilder", "BatchConfig", "Batcher"]


class TrainingSampleBuilder(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        drop_zero_std_reward_groups: bool = True

    def __init__(self, config: Config | None = None, **_):
        self.config = config or TrainingSampleBuilder.Config()

    def build_from_group(self, *, rollout_group: RolloutGroup) -> TrainingSampleGroup:
        g = rollout_group
        metrics = list(g.metrics)

        def empty():
            return TrainingSampleGroup(group_id=g.group_id, training_samples=[], metrics=metrics)

        if not g.rollouts:
            return empty()
        if any(not any(t.completion_token_ids for t in r.turns) for r in g.rollouts):
            metrics.append(m.Metric("training_sample_builder/num_groups_dropped_untrainable", m.Sum(1.0)))
            return empty()
        rewards = [r.reward for r in g.rollouts]
        zero_std = len(rewards) > 1 and statistics.pstdev(rewards) == 0.0
        metrics.append(m.Metric("rollout_reward/group_zero_std_frac", m.Mean(1.0 if zero_std else 0.0)))
        if zero_std and self.config.drop_zero_std_reward_groups:
            metrics.append(m.Metric("training_sample_builder/num_groups_dropped_zero_std", m.Sum(1.0)))
            return empty()
        samples, branches = [], []
        for r in g.rollouts:
            s = self.rollout_to_training_samples(r)
            samples += s
            branches.append(float(len(s)))
        metrics += [
            m.Metric("training_sample_builder/num_training_samples", m.Sum(float(len(samples)))),
            m.Metric("advantage", m.SummaryStats.from_list([r.advantage for r in g.rollouts])),
            m.Metric("rollout/branches_per_rollout", m.Mean.from_list(branches)),
            m.Metric("rollout/branches_per_rollout", m.Max.from_list(branches)),
            m.Metric("rollout/min_policy_version", m.Min.from_list([s.min_policy_version for s in samples])),
            m.Metric("rollout/max_policy_version", m.Max.from_list([s.max_policy_version for s in samples])),
        ]
        return TrainingSampleGroup(group_id=g.group_id, training_samples=samples, metrics=metrics)

    def rollout_to_training_samples(self, rollout: Rollout) -> list[TrainingSample]:
        """Example (P prompt, C completion, E environment reply; the environment compacts history before turn 3)::

            turn0 prompt=[P1]             completion=[C1]   \\
            turn1 prompt=[P1,C1,E1]       completion=[C2]    > sample 0 = P1 C1 E1 C2 E2 C3, trained on C1 C2 C3
            turn2 prompt=[P1,C1,E1,C2,E2] completion=[C3]   /
            turn3 prompt=[P2]             completion=[C4]   \\  sample 1 = P2 C4 E4 C5, trained on C4 C5
            turn4 prompt=[P2,C4,E4]       completion=[C5]   /

        A sample's ``min_policy_version`` is that of its first turn (what the off-policy accounting reads), its
        ``max_policy_version`` the newest any of its turns saw."""
        adv = rollout.advantage
        if adv is None:
            raise ValueError(f"rollout {rollout.group_id}/{rollout.rollout_id} has no advantage: the rollouter's "
                             "advantage estimator must run before samples are built")
        out: list[TrainingSample] = []
        prev: list[int] = []
        for i, t in enumerate(rollout.turns):
            if not t.completion_token_ids:
                if len(rollout.turns) == 1:
                    continue
                raise ValueError(f"rollout {rollout.group_id}/{rollout.rollout_id}: turn {i} has no completion")
            prompt = t.prompt_token_ids
            if not out or prompt[:len(prev)] != prev:
                out.append(TrainingSample(
                    rollout_id=RolloutTurnID(group_id=rollout.group_id, rollout_id=rollout.rollout_id, turn_id=i),
                    min_policy_version=t.min_policy_version, max_policy_version=t.max_policy_version,
                    token_ids=[], loss_mask=[], logprobs=[], advantage=[]))
                start = 0
            else:
                start = len(prev)
            s = out[-1]
            delta, n = prompt[start:], len(t.completion_token_ids)
            s.token_ids += delta + list(t.completion_token_ids)
            s.loss_mask += [False] * len(delta) + [True] * n
            s.logprobs += [0.0] * len(delta) + list(t.completion_logprobs)
            s.advantage += [0.0] * len(delta) + [adv] * n
            s.max_policy_version = max(s.max_policy_version, t.max_policy_version)
            prev = list(prompt) + list(t.completion_token_ids)
        return out


@dataclass(kw_only=True, slots=True)
class BatchConfig:
    local_batch_size: int = 8
    """Rows per data-parallel rank and microbatch."""
    seq_len: int = 2048
    """Tokens per packed row."""


_FIELDS = {"input_ids": torch.long, "labels": torch.long, "generator_logprobs": torch.float32, "loss_mask": torch.bool,
           "advantages": torch.float32}


class Batcher(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        batch: BatchConfig = field(default_factory=BatchConfig)
        per_sample_pad_multiple: int | None = None
        """Pad every sample to a multiple of this many tokens before packing (batch-invariant mode: attention
        block boundaries then do not depend on what else is in the row)."""

    def __init__(self, config: Config | None = None, *, num_prompts_per_train_step: int, dp_degree: int, pad_id: int):
        self.config = config or Batcher.Config()
        self.local_batch_size, self.seq_len = self.config.batch.local_batch_size, self.config.batch.seq_len
        self.pad_id = pad_id
        self._pad_to = self.config.per_sample_pad_multiple
        self._need, self._dp = num_prompts_per_train_step, dp_degree
        self._pending: list[TrainingSampleGroup] = []

    # -- accumulation --------------------------------------------------------------------------------------------
    def num_tokens_to_pack(self, s: TrainingSample) -> int:
        n = len(s.token_ids) - 1                 # the input / label split drops one token
        return n if not self._pad_to else (n + self._pad_to - 1) // self._pad_to * self._pad_to

    def add_training_samples(self, *, training_sample_group: TrainingSampleGroup) -> TrainingBatch | None:
        """Returns a batch once ``num_prompts_per_train_step`` trainable groups have accumulated (groups without
        samples only carry their metrics along), else ``None``."""
        g = training_sample_group
        kept = [s for s in g.training_samples if self.num_tokens_to_pack(s) <= self.seq_len]
        if len(kept) != len(g.training_samples):
            dropped = len(g.training_samples) - len(kept)
            logger.warning(f"batcher dropped {dropped}/{len(g.training_samples)} sample(s) longer than seq_len={self.seq_len}")
            g = dataclasses.replace(g, training_samples=kept, metrics=[
                *g.metrics, m.Metric("batcher/num_samples_dropped_oversized", m.Sum(float(dropped)))])
        self._pending.append(g)
        if sum(bool(x.training_samples) for x in self._pending) < self._need:
            return None
        return self._pack()

    def _pack(self) -> TrainingBatch:
        samples, metrics, trainable, cut = [], [], 0, 0
        for g in self._pending:                 # oldest first
            if trainable >= self._need:
                break
            cut += 1
            metrics += g.metrics
            if g.training_samples:
                trainable += 1
                samples += g.training_samples
        self._pending = self._pending[cut:]
        rows = [self._pack_row(r) for r in self._assign_rows(samples)]
        valid = sum(int((r["loss_mask"] & torch.isfinite(r["generator_logprobs"])).sum()) for r in rows)
        response = sum(int(r["loss_mask"].sum()) for r in rows)
        real = sum(sum(r["seq_lens"]) for r in rows)
        grid = self._grid(rows)                  # appends pad-only rows
        slots = len(rows) * self.seq_len
        metrics += [
            m.Metric("loss/generator_logprob_nan_frac", m.NoReduce((response - valid) / max(response, 1))),
            m.Metric("train_batch/padding_frac", m.NoReduce((slots - real) / slots)),
            m.Metric("train_batch/num_microbatches", m.NoReduce(float(len(grid)))),
            m.Metric("train_batch/num_rollout_groups", m.NoReduce(float(trainable))),
            m.Metric("train_batch/num_metric_only_groups", m.NoReduce(float(cut - trainable))),
            m.Metric("train_batch/num_training_samples", m.NoReduce(float(len(samples)))),
        ]
        return TrainingBatch(microbatches=grid, num_global_valid_tokens=valid, metrics=metrics,
                             min_policy_versions=[s.min_policy_version for s in samples])

    # -- packing -------------------------------------------------------------------------------------------------
    def _assign_rows(self, samples: list[TrainingSample]) -> list[list[TrainingSample]]:
        rows, cur, used = [], [], 0
        for s in samples:                        # next fit: order (and with it sibling adjacency) is kept
            n = self.num_tokens_to_pack(s)
            if cur and used + n > self.seq_len:
                rows.append(cur)
                cur, used = [], 0
            cur.append(s)
            used += n
        if cur:
            rows.append(cur)
        return rows

    def _pack_row(self, samples: list[TrainingSample]) -> dict:
        pad = {"input_ids": self.pad_id, "labels": self.pad_id, "generator_logprobs": 0.0, "loss_mask": False,
               "advantages": 0.0}
        row: dict[str, list] = {k: [] for k in _FIELDS}
        positions: list[int] = []
        seq_lens: list[int] = []
        for s in samples:
            part = {"input_ids": s.token_ids[:-1], "labels": s.token_ids[1:], "generator_logprobs": s.logprobs[1:],
                    "loss_mask": s.loss_mask[1:], "advantages": s.advantage[1:]}
            n = len(part["input_ids"])
            full = self.num_tokens_to_pack(s)
            for k in _FIELDS:
                row[k] += list(part[k]) + [pad[k]] * (full - n)
            positions += range(full)
            seq_lens.append(full)
        tail = self.seq_len - len(positions)
        for k in _FIELDS:
            row[k] += [pad[k]] * tail
        positions += range(tail)                 # the padding is one more (masked) document
        out = {k: torch.tensor(row[k], dtype=dt) for k, dt in _FIELDS.items()}
        out["positions"] = torch.tensor(positions, dtype=torch.long)
        out["seq_lens"] = seq_lens
        return out

    def _grid(self, rows: list[dict]) -> list[list[TrainingMicrobatch]]:
        per_mb = self.local_batch_size * self._dp
        n_mb = max(1, math.ceil(len(rows) / per_mb))
        while len(rows) < n_mb * per_mb:
            rows.append(self._pack_row([]))
        stride = n_mb * self._dp                 # round-robin: the pad-only rows at the end spread over all cells
        return [[self.collate(rows[mb * self._dp + rank::stride]) for rank in range(self._dp)] for mb in range(n_mb)]

    @staticmethod
    def collate(rows: list[dict]) -> TrainingMicrobatch:
        cat = lambda k: torch.cat([r[k] for r in rows])   # noqa: E731
        return TrainingMicrobatch(token_ids=cat("input_ids"), labels=cat("labels"), positions=cat("positions"),
                                  generator_logprobs=cat("generator_logprobs"), loss_mask=cat("loss_mask"),
                                  advantages=cat("advantages"))
