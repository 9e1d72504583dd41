"""The training side of the asynchronous RL loop: packed microbatches in, policy versions out.

``PolicyTrainer`` wraps a parallelised decoder, its sharding engine and optimizers.  ``forward_backward`` takes the
``[dp rank]`` row of a ``TrainingBatch`` microbatch grid, runs this rank's flat microbatch (documents kept apart by
the position restarts) and accumulates gradients; ``optim_step`` clips, steps, advances the LR schedule and bumps
``policy_version``; ``push_model_state_dict`` makes the new weights readable for the generators' pull (it joins the
optimizer that overlaps with the next forward).

Parity: torchtitan/experiments/rl/actors/trainer.py:47-527 (there a Monarch actor mesh; here an object of the
training ranks, driven from the controller's event loop).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .losses import PolicyLoss
from .records import OptimStepOutput, TrainingMicrobatch

__all__ = ["PolicyTrainer"]


class PolicyTrainer:
    def __init__(self, *, model, engine, optimizers, loss: PolicyLoss | None = None, pdims=None, lr_schedulers=None,
                 max_norm: float = 1.0, start_version: int = 0):
        self.model, self.engine, self.optimizers = model, engine, optimizers
        self.loss = loss or PolicyLoss()
        self.pdims, self.lr_schedulers, self.max_norm = pdims, lr_schedulers, max_norm
        self.policy_version = start_version
        self._accumulating = False

    @property
    def dp_rank(self) -> int:
        return self.pdims.dp_rank if self.pdims is not None and hasattr(self.pdims, "dp_rank") else 0

    def forward_backward(self, microbatch_row: list[TrainingMicrobatch], num_global_valid_tokens: int) -> dict[str, float]:
        if not self._accumulating:
            self.optimizers.zero_grad()
            self._accumulating = True
        mb = microbatch_row[self.dp_rank if len(microbatch_row) > 1 else 0]
        dev = next(self.model.parameters()).device
        tokens, positions, labels = mb.token_ids.to(dev), mb.positions.to(dev), mb.labels.to(dev)
        logits = self.model(tokens, positions)
        loss, stats = self.loss(logits, labels, num_global_valid_tokens, generator_logprobs=mb.generator_logprobs.to(dev),
                                advantages=mb.advantages.to(dev), loss_mask=mb.loss_mask.to(dev))
        del logits
        loss.backward()
        self.engine.finish_backward()
        keys = sorted(stats)
        vec = torch.stack([stats[k].float().reshape(()) for k in keys])
        group = self.pdims.group("loss") if self.pdims is not None and dist.is_initialized() else None
        if group is not None:
            mx = [i for i, k in enumerate(keys) if k.endswith("/max")]
            top = vec[mx].clone()
            dist.all_reduce(vec, group=group)
            if mx:
                dist.all_reduce(top, op=dist.ReduceOp.MAX, group=group)
                vec[mx] = top
        return dict(zip(keys, vec.cpu().tolist()))

    def optim_step(self) -> OptimStepOutput:
        from torchtitan_b200.components.optimizer import clip_grad_norm_

        norm = clip_grad_norm_([self.engine], self.max_norm, self.pdims, optimizers=self.optimizers)
        self.optimizers.step()
        stats = {"optim/grad_norm": float(norm)}
        if self.lr_schedulers is not None:
            self.lr_schedulers.step()
            stats.update({f"optim/{k}": float(v) for k, v in self.lr_schedulers.get_metrics().items()})
        self._accumulating = False
        self.policy_version += 1
        return OptimStepOutput(policy_version=self.policy_version, metrics=stats)

    def push_model_state_dict(self) -> None:
        if hasattr(self.engine, "wait_optimizer"):
            self.engine.wait_optimizer()
