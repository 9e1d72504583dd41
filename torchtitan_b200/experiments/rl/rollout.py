"""SampledResponse records and a FIFO buffer that folds them into training batches."""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass

import torch

__all__ = ["SampledResponse", "RolloutBuffer"]


@dataclass
class SampledResponse:
    prompt: torch.Tensor       # [P] token ids
    response: torch.Tensor     # [R] token ids
    logprobs: torch.Tensor     # [R] behaviour-policy log-probabilities of the response tokens
    reward: float = 0.0
    policy_version: int = 0


class RolloutBuffer:
    def __init__(self, max_size: int = 4096, max_staleness: int = 1):
        self.items: deque[SampledResponse] = deque(maxlen=max_size)
        self.max_staleness = max_staleness

    def add(self, rollouts) -> None:
        self.items.extend(rollouts)

    def evict_stale(self, current_version: int) -> int:
        keep = [r for r in self.items if current_version - r.policy_version <= self.max_staleness]
        dropped = len(self.items) - len(keep)
        self.items = deque(keep, maxlen=self.items.maxlen)
        return dropped

    def fold(self, rollouts: list[SampledResponse], advantages: torch.Tensor):
        """Concatenate samples into one token stream: ``(tokens, positions, labels, old_logp, adv, mask)``.
        Position restarts at every sample (document masking keeps samples apart); labels are the next
        token, prompt positions and the last token of each sample are masked out."""
        toks, pos, lab, old, adv, mask = [], [], [], [], [], []
        for r, a in zip(rollouts, advantages.tolist()):
            seq = torch.cat([r.prompt, r.response])
            n, p = seq.numel(), r.prompt.numel()
            toks.append(seq)
            pos.append(torch.arange(n))
            lab.append(torch.cat([seq[1:], seq.new_full((1,), -100)]))
            m = torch.zeros(n)
            m[p - 1:n - 1] = 1.0                      # token t predicts t + 1: response targets
            o = torch.zeros(n)
            o[p - 1:n - 1] = r.logprobs.float()
            old.append(o)
            mask.append(m)
            adv.append(torch.full((n,), float(a)))
        cat = torch.cat
        return cat(toks), cat(pos), cat(lab), cat(old), cat(adv), cat(mask)
