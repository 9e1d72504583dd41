"""Periodic validation on a separate dataloader.

Loss = sum over valid tokens / global valid tokens, reduced over the ``loss`` mesh;
``steps = -1`` consumes one finite pass of the validation set.  Parity:
torchtitan/components/validate.py:34-356.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from torchtitan_b200.components.data import BaseDataLoader
from torchtitan_b200.components.loss import IGNORE_INDEX
from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

__all__ = ["Validator"]


class Validator(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        enable: bool = False
        freq: int = 10
        steps: int = -1
        dataloader: BaseDataLoader.Config = field(
            default_factory=lambda: BaseDataLoader.Config(dataset="c4_validation", repeat=False, shuffle=False))

    def __init__(self, config: "Validator.Config", *, trainer, **_):
        self.config = config
        self.trainer = trainer
        t = trainer
        self.dataloader = config.dataloader.build(
            dp_world_size=t.pdims.dp_degree, dp_rank=t.pdims.dp_rank,
            num_tokens_per_batch=t.config.training.num_tokens_per_microbatch_per_dp_rank,
            max_context_length=t.config.training.max_context_length, vocab_size=t.model_config.vocab_size,
            tokenizer=t.tokenizer)
        if config.steps == -1 and config.dataloader.repeat:
            logger.warning("validator.steps=-1 with a repeating dataloader never terminates; set repeat=False")

    def should_validate(self, step: int) -> bool:
        return step == 1 or step % self.config.freq == 0

    @torch.no_grad()
    def validate(self, model_parts, step: int) -> float:
        t = self.trainer
        pd = t.pdims
        for m in model_parts:
            m.eval()
        total = torch.zeros((), dtype=torch.float32, device=t.device)
        ntok = torch.zeros((), dtype=torch.float32, device=t.device)
        n = 0
        n_mb = t.config.parallelism.num_pp_microbatches if pd.pp_enabled else 1
        pending: list = []
        for inputs, labels in self.dataloader:
            if 0 < self.config.steps <= n:
                break
            t.metrics_processor.ntokens_since_last_log += labels.numel()
            one = torch.ones((), dtype=torch.float32, device=t.device)
            if pd.pp_enabled:
                from torchtitan_b200.parallel.pipeline import run_pipeline_eval

                pending.append((inputs, labels))
                if len(pending) < n_mb:
                    continue
                stacked = {k: torch.stack([p[0][k] for p in pending]) for k in pending[0][0]}
                slab = torch.stack([p[1] for p in pending])
                pending = []
                tokens, positions, lab, q_pos = t.post_dataloading_process(stacked, slab)
                loss = run_pipeline_eval(t, tokens, positions, lab, q_pos)
            else:
                tokens, positions, lab, q_pos = t.post_dataloading_process(inputs, labels)
                model = t.model
                ctx = model.build_context(positions, q_pos)
                pred = model(tokens, positions, ctx, return_hidden=t.loss_fn.needs_hidden)
                loss = t.loss_fn(pred, lab, one)
            total += loss.float()
            ntok += (lab != IGNORE_INDEX).sum()
            n += 1
        stats = torch.stack([total, ntok])
        g = pd.group("loss")
        if g is not None:
            dist.all_reduce(stats, group=g)
        if pd.pp_enabled:
            dist.all_reduce(stats[:1], group=pd.group("pp"))
            dist.all_reduce(stats[1:], op=dist.ReduceOp.MAX, group=pd.group("pp"))
        loss = (stats[0] / stats[1].clamp_min(1.0)).item()
        t.metrics_processor.log_validation(loss, step)
        for m in model_parts:
            m.train()
        return loss
