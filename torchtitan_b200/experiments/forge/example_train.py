"""A training loop written against :class:`ForgeEngine`'s verbs, the way an external framework would drive it.

    python -m torchtitan_b200.experiments.forge.example_train --module llama3 --config llama3_debugmodel \\
        --training.steps 20

``ExampleTrainer`` owns the loop that ``ForgeEngine`` deliberately lacks: it pulls microbatches from the engine's
dataloader, counts the step's valid tokens over the data-parallel group, calls ``forward_backward`` per microbatch and
``optimizer_step`` once, logs through the engine's metrics processor, saves through its checkpoint manager and
resumes from it.  Parity: torchtitan/experiments/forge/example_train.py:31-476 (a trainer subclassing the engine).
"""

from __future__ import annotations

import sys
import time

import torch
import torch.distributed as dist

from torchtitan_b200.components.loss import IGNORE_INDEX
from torchtitan_b200.utils.logging import init_logger, logger

from .engine import ForgeEngine

__all__ = ["ExampleTrainer", "main"]


class ExampleTrainer(ForgeEngine):
    def train_step(self, data_iterator) -> tuple[float, float]:
        """One optimizer step over ``gradient_accumulation_steps`` microbatches; returns (loss, gradient norm)."""
        micro = [next(data_iterator) for _ in range(self.gradient_accumulation_steps)]
        valid = torch.tensor([float(sum(int((lab != IGNORE_INDEX).sum()) for _, lab in micro))], device=self.device)
        group = self.pdims.group("batch")
        if group is not None:
            dist.all_reduce(valid, group=group)
        loss = torch.zeros((), device=self.device)
        for inputs, labels in micro:
            loss = loss + self.forward_backward(inputs["input"], labels, positions=inputs.get("positions"),
                                                global_valid_tokens=float(valid)).reshape(())
            self.ntokens_seen += labels.numel() * self.pdims.dp_degree
        norm = self.optimizer_step()
        lg = self.pdims.group("loss")
        if lg is not None:
            dist.all_reduce(loss, group=lg)
        return float(loss), float(norm)

    def train(self) -> list[float]:
        c = self.config
        self.load()                      # resumes when the checkpoint folder holds a step, otherwise a no-op
        it = self.batch_generator(self.dataloader)
        losses = []
        t0 = time.perf_counter()
        while self.step < c.training.steps:
            loss, norm = self.train_step(it)
            losses.append(loss)
            if self.step % max(1, c.metrics.log_freq) == 0 or self.step == c.training.steps:
                dt = time.perf_counter() - t0
                logger.info(f"[forge example] step {self.step:4d}  loss {loss:8.4f}  grad norm {norm:7.3f}  "
                            f"{dt:6.2f} s since the last log")
                t0 = time.perf_counter()
            if c.checkpoint.enable and self.step % max(1, c.checkpoint.interval) == 0:
                self.save(self.step, last_step=self.step == c.training.steps)
        return losses


def main(argv: list[str] | None = None, trainer_cls: type[ExampleTrainer] = ExampleTrainer) -> list[float]:
    from torchtitan_b200.config import ConfigManager

    init_logger()
    cfg = ConfigManager().parse_args(sys.argv[1:] if argv is None else argv)
    trainer = trainer_cls(cfg)
    try:
        return trainer.train()
    finally:
        trainer.close()


if __name__ == "__main__":
    main()
