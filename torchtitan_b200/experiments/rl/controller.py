"""The RL post-training loop: rollouts -> rewards -> group-relative advantages -> policy-gradient step ->
weight push (parity: torchtitan/experiments/rl/controller.py and train.py, which drive a trainer actor and
generator actors; here both are objects of one process or ranks of one job).

One iteration of ``RLController.step``:

1. every prompt is answered ``group_size`` times by the generator (behaviour policy, cached decoding);
2. ``reward_fn(prompt, response) -> float`` scores each answer; groups whose answers all score the same carry no
   signal and are dropped when ``dynamic_sampling`` is on (DAPO's filter);
3. advantages are normalised inside each group; samples older than ``max_staleness`` policy versions are evicted;
4. the samples are folded into one token stream (documents keep them apart), the policy's token log-probabilities
   come from the training model, and the GRPO or DAPO surrogate is minimised with the sharded optimizer;
5. every ``sync_every`` iterations the new weights are pushed to the generator.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from .generator import SamplingGenerator, WeightSync
from .losses import dapo_loss, group_advantages, grpo_loss, token_logprobs
from .rollout import SampledResponse, RolloutBuffer

__all__ = ["RLConfig", "RLController"]


@dataclass
class RLConfig:
    group_size: int = 4
    max_new_tokens: int = 16
    loss: str = "grpo"            # grpo | dapo
    clip_eps: float = 0.2
    clip_eps_high: float = 0.28   # DAPO's upper clip range
    kl_coef: float = 0.0
    dynamic_sampling: bool = False
    sync_every: int = 1
    max_staleness: int = 1


class RLController:
    def __init__(self, model, engine, optimizers, generator: SamplingGenerator, reward_fn: Callable, config: RLConfig,
                 *, pdims=None, ref_model=None, weight_sync: WeightSync | None = None):
        self.model, self.engine, self.optimizers = model, engine, optimizers
        self.generator, self.reward_fn, self.cfg = generator, reward_fn, config
        self.pdims = pdims
        self.ref_model = ref_model
        self.sync = weight_sync or WeightSync()
        self.buffer = RolloutBuffer(max_staleness=config.max_staleness)
        self.iteration = 0

    def collect(self, prompts: list[torch.Tensor]) -> tuple[list[SampledResponse], torch.Tensor]:
        c = self.cfg
        rollouts, rewards = [], []
        self._all_rewards: list[float] = []
        for prompt in prompts:
            group = [self.generator.generate(prompt, c.max_new_tokens) for _ in range(c.group_size)]
            r = [float(self.reward_fn(g.prompt, g.response)) for g in group]
            self._all_rewards += r
            if c.dynamic_sampling and max(r) == min(r):
                continue                      # no learning signal in this group
            for g, ri in zip(group, r):
                g.reward = ri
            rollouts += group
            rewards += r
        return rollouts, torch.tensor(rewards)

    def step(self, prompts: list[torch.Tensor]) -> dict:
        from torchtitan_b200.components.optimizer import clip_grad_norm_

        c = self.cfg
        rollouts, rewards = self.collect(prompts)
        # the reward of everything that was generated, the groups dropped by dynamic sampling included
        stats = {"reward_mean": sum(self._all_rewards) / max(1, len(self._all_rewards)), "samples": len(rollouts)}
        self.buffer.evict_stale(self.sync.version)
        if not rollouts:
            return stats
        adv = group_advantages(rewards, c.group_size)
        tokens, positions, labels, old_logp, adv_t, mask = self.buffer.fold(rollouts, adv)
        dev = next(self.model.parameters()).device
        tokens, positions, old_logp, adv_t, mask = (t.to(dev) for t in (tokens, positions, old_logp, adv_t, mask))
        targets = labels.to(dev).clamp_min(0)
        self.optimizers.zero_grad()
        logits = self.model(tokens, positions)
        logp, entropy = token_logprobs(logits, targets)
        ref_logp = None
        if self.ref_model is not None and c.kl_coef:
            with torch.no_grad():
                ref_logp, _ = token_logprobs(self.ref_model(tokens, positions), targets, with_entropy=False)
        if c.loss == "dapo":
            loss, extra = dapo_loss(logp, old_logp, adv_t, mask, eps_low=c.clip_eps, eps_high=c.clip_eps_high)
        else:
            loss, extra = grpo_loss(logp, old_logp, adv_t, mask, ref_logp=ref_logp, clip_eps=c.clip_eps, kl_coef=c.kl_coef)
        loss.backward()
        self.engine.finish_backward()
        clip_grad_norm_([self.engine], 1.0, self.pdims, optimizers=self.optimizers)
        self.optimizers.step()
        self.iteration += 1
        if self.iteration % c.sync_every == 0 and self.generator.model is not self.model:
            self.sync.push(self.model, self.generator, engine=self.engine)
        elif self.generator.model is self.model:
            self.sync.version += 1
            self.generator.policy_version = self.sync.version
        stats.update(loss=float(loss.detach()), entropy=float((entropy.detach() * mask).sum() / mask.sum().clamp_min(1)), **extra)
        return stats
