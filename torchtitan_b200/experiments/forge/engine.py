"""Engine object without a training loop.

``ForgeEngine(config)`` performs everything ``Trainer.__init__`` does (process group, mesh, model
on the meta device, parallelisation, sharded-parameter engine, optimizer, LR schedule, checkpoint
manager) and exposes the pieces plus three verbs for callers that own the loop:

    loss = engine.forward_backward(tokens, labels)     # one microbatch, gradients accumulate
    norm = engine.optimizer_step()                     # reduce-scatter, clip, AdamW, LR step
    engine.save(step) / engine.load()
"""

from __future__ import annotations

import torch

from torchtitan_b200.components.optimizer import clip_grad_norm_
from torchtitan_b200.trainer import Trainer

__all__ = ["ForgeEngine"]


class ForgeEngine(Trainer):
    Config = Trainer.Config

    def __init__(self, config: Trainer.Config, **kw):
        super().__init__(config, **kw)
        self._zeroed = False

    def forward_backward(self, tokens: torch.Tensor, labels: torch.Tensor, *, positions: torch.Tensor | None = None,
                         global_valid_tokens: float | None = None) -> torch.Tensor:
        """One microbatch of folded tokens ``[T]``; returns the (sum / global tokens) loss."""
        if not self._zeroed:
            self.optimizers.zero_grad()
            self._zeroed = True
        tokens = tokens.to(self.device)
        labels = labels.to(self.device)
        if positions is None:
            positions = torch.arange(tokens.shape[0], device=self.device)
        n = float((labels != -100).sum()) if global_valid_tokens is None else float(global_valid_tokens)
        valid = torch.tensor([max(n, 1.0)], dtype=torch.float32, device=self.device)
        return self.forward_backward_step({"input": tokens, "positions": positions.to(self.device)}, labels, valid)

    def optimizer_step(self) -> torch.Tensor:
        norm = clip_grad_norm_(self.engines, self.config.training.max_norm, self.pdims, optimizers=self.optimizers)
        self.optimizers.step()
        self.lr_schedulers.step()
        self.step += 1
        self._zeroed = False
        return norm

    def save(self, step: int | None = None, last_step: bool = False) -> None:
        self.checkpointer.save(self.step if step is None else step, last_step=last_step)

    def load(self, step: int = -1) -> bool:
        return self.checkpointer.load(step=step)

    def train(self) -> None:  # pragma: no cover - by design
        raise RuntimeError("ForgeEngine has no training loop; drive forward_backward / optimizer_step yourself")
