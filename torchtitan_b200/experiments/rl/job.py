"""One RL job: the training ranks, the generators and the controller, built from one config.

``RLJob.Config`` holds a full ``Trainer.Config`` (model, parallelism, optimizer, schedule, checkpointing: the
policy is trained by the same engine as pre-training, built through ``ForgeEngine``), the generation engine's
config and the controller's.  Placement:

* ``share_weights = True`` (default): one generation engine on the training model object itself.  In the resident
  FSDP layout every rank holds the full bf16 weights, refreshed by the optimizer kernel, so nothing is copied for a
  "weight sync"; generation and training alternate on the device.
* ``share_weights = False``: ``num_generators`` engines, each with its own copy of the model on
  ``generator_devices[i]`` (other GPUs of the node), running in worker threads while the trainer trains; a pull
  copies the trainer's parameters device to device.

The trainer is data-parallel (FSDP / HSDP) with the resident parameter layout; other layouts are refused at start,
because a generator runs the whole model on one device.  With more than one training rank the controller lives on rank 0; it announces every trainer call to the other
ranks (``_LeaderTrainer`` / ``follow``), which run the same call on their shard of the microbatch grid.

Parity: torchtitan/experiments/rl/train.py:46-314 and controller.py:261-520 (setup: Monarch proc meshes for the
trainer and each generator, TorchStore for the weights).
"""

from __future__ import annotations

import asyncio
import json
import os
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

from torchtitan_b200.config import Configurable
from torchtitan_b200.trainer import Trainer
from torchtitan_b200.utils.logging import logger

from .async_controller import AsyncController
from .engine import GenerationEngine, place_model_
from .losses import PolicyLoss
from .policy_trainer import PolicyTrainer

__all__ = ["RLJob"]


def _announce(msg: Any) -> Any:
    box = [msg]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class _LeaderTrainer(PolicyTrainer):
    """Rank 0's trainer: every call is first announced to the follower ranks, which then join its collectives."""

    def forward_backward(self, row, n):
        _announce(("forward_backward", row, n))
        return super().forward_backward(row, n)

    def optim_step(self):
        _announce(("optim_step",))
        return super().optim_step()

    def push_model_state_dict(self):
        _announce(("push",))
        return super().push_model_state_dict()

    def save(self, forge, step, last):
        _announce(("save", step, last))
        forge.step = step
        forge.save(step, last_step=last)


def follow(trainer: PolicyTrainer, forge) -> None:
    """The loop of every training rank but 0."""
    while True:
        op, *args = _announce(None)
        if op == "stop":
            return
        if op == "forward_backward":
            trainer.forward_backward(*args)
        elif op == "optim_step":
            trainer.optim_step()
        elif op == "push":
            trainer.push_model_state_dict()
        elif op == "save":
            forge.step = args[0]
            forge.save(args[0], last_step=args[1])


class RLJob(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        trainer: Trainer.Config
        controller: AsyncController.Config
        generator: GenerationEngine.Config = field(default_factory=GenerationEngine.Config)
        num_generators: int = 1
        share_weights: bool = True
        generator_devices: list[str] = field(default_factory=list)
        """Devices of the generator replicas when they hold their own weights (default: the trainer's device)."""
        ratio_clip_low: float = 0.2
        ratio_clip_high: float = 0.2
        """Larger than ``ratio_clip_low``: DAPO's clip-higher."""
        byte_tokenizer: bool = False
        """Use the built-in byte tokenizer instead of the files under ``trainer.hf_assets_path``."""

        def validate(self) -> None:
            t = self.trainer
            if self.num_generators < 1:
                raise ValueError(f"num_generators must be >= 1, got {self.num_generators}")
            if self.share_weights and self.num_generators != 1:
                raise ValueError("share_weights runs exactly one generator on the training model")
            if t.parallelism.fsdp_reshard_after_forward == "always":
                raise ValueError("the RL job needs the resident parameter layout: the generators read (or copy) the "
                                 "trainer's full weights between optimizer steps")
            par = t.parallelism
            if max(par.pipeline_parallel_degree, par.context_parallel_degree, par.tensor_parallel_degree,
                   par.expert_parallel_degree) > 1:
                # the generators run the whole model on one device: with shared weights rank 0 generates alone (layers
                # that need their tensor- / expert-parallel peers cannot), with own copies the pull copies full tensors
                raise ValueError("the RL job trains with data parallelism (FSDP / HSDP); tensor, expert, context and "
                                 "pipeline parallelism are not supported here")
            b = self.controller.async_loop.batcher.batch
            # the batcher's grid decides the training shapes
            t.training.max_context_length = b.seq_len
            t.training.num_tokens_per_microbatch_per_dp_rank = b.seq_len * b.local_batch_size
            t.training.num_tokens_per_train_step = -1
            t.dataloader.dataset = "synthetic"
            env = self.controller.rollouter.token_env
            if env.max_rollout_tokens is None:
                # a conversation that no longer fits a packed row ends as "truncated_prompt_too_long" instead of failing
                # in the generator
                env.max_rollout_tokens = b.seq_len - 1
            if self.share_weights:
                self.generator.threaded = False
                self.controller.trainer_in_thread = False
            if callable(getattr(t, "validate", None)):
                t.validate()

    def __init__(self, config: Config, **_):
        from torchtitan_b200.experiments.forge import ForgeEngine

        self.config = config
        self.forge = forge = ForgeEngine(config.trainer)
        if any(getattr(e, "sharded_params", False) for e in forge.engines):
            raise ValueError("the sharding engine chose the sharded parameter layout for this model; the RL job needs "
                             "full weights between steps: set parallelism.fsdp_reshard_after_forward = never")
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        cls = _LeaderTrainer if dist.is_initialized() and dist.get_world_size() > 1 and self.rank == 0 else PolicyTrainer
        self.trainer = cls(model=forge.model, engine=forge.engines[0], optimizers=forge.optimizers,
                           lr_schedulers=forge.lr_schedulers, pdims=forge.pdims, max_norm=config.trainer.training.max_norm,
                           loss=PolicyLoss(config.ratio_clip_low, config.ratio_clip_high))
        resumed = bool(config.trainer.checkpoint.enable and forge.load())
        if resumed:
            self.trainer.policy_version = forge.step
        self.controller = None
        if self.rank != 0:
            return
        if config.byte_tokenizer or not os.path.isdir(config.trainer.hf_assets_path):
            from torchtitan_b200.components.tokenizer import ByteTokenizer

            tokenizer = ByteTokenizer()
        else:
            from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer

            tokenizer = HuggingFaceTokenizer(tokenizer_path=config.trainer.hf_assets_path)
        if tokenizer.get_vocab_size() > forge.model_config.vocab_size:
            raise ValueError(f"the tokenizer has {tokenizer.get_vocab_size()} tokens, the model {forge.model_config.vocab_size}")
        self.generators = self._build_generators(tokenizer)
        self.controller = AsyncController(config.controller, trainer=self.trainer, generators=self.generators,
                                          tokenizer=tokenizer, dp_degree=forge.pdims.dp_degree,
                                          step_callback=self._after_step if config.trainer.checkpoint.enable else None)
        self.controller.start_step = self.trainer.policy_version
        for g in self.generators:
            g.policy_version = self.trainer.policy_version
        self._state_path = os.path.join(config.trainer.dump_folder, config.trainer.checkpoint.folder, "rl_state.json")
        if resumed and os.path.exists(self._state_path):
            with open(self._state_path) as f:
                state = json.load(f)
            if state.get("policy_version") == self.trainer.policy_version:
                self.controller.rollouter.load_dataset_state(state.get("datasets", {}))
                logger.info(f"RL job resumed at policy version {self.trainer.policy_version} with its dataset position")

    def _after_step(self, step: int, last: bool) -> None:
        """Checkpoint at the trainer's interval: model / optimizer / schedule through the regular checkpoint manager,
        plus the datasets' positions (prompt groups still in flight at the save are regenerated after a resume)."""
        c = self.config.trainer.checkpoint
        if not (last or step % max(c.interval, 1) == 0):
            return
        if isinstance(self.trainer, _LeaderTrainer):
            self.trainer.save(self.forge, step, last)
        else:
            self.forge.step = step
            self.forge.save(step, last_step=last)
        os.makedirs(os.path.dirname(self._state_path), exist_ok=True)
        with open(self._state_path + ".tmp", "w") as f:
            json.dump({"policy_version": step, "datasets": self.controller.rollouter.dataset_state()}, f)
        os.replace(self._state_path + ".tmp", self._state_path)

    def _build_generators(self, tokenizer) -> list[GenerationEngine]:
        c, forge = self.config, self.forge
        eos = int(tokenizer.eos_id) if tokenizer.eos_id is not None else None
        if c.share_weights:
            return [c.generator.build(model=forge.model, eos_id=eos)]
        out = []
        for i in range(c.num_generators):
            dev = torch.device(c.generator_devices[i] if i < len(c.generator_devices) else forge.device)
            copy = place_model_(forge.model_config.build(), dev, next(forge.model.parameters()).dtype)
            if hasattr(copy, "init_buffers"):
                copy.init_buffers(dev)
            out.append(c.generator.build(model=copy, eos_id=eos, weight_source=self._copy_weights))
            self._copy_weights(out[-1])
        return out

    @torch.no_grad()
    def _copy_weights(self, engine: GenerationEngine) -> None:
        src = dict(self.forge.model.named_parameters())
        for name, p in engine.model.named_parameters():
            p.copy_(src[name].detach().to(p.device, p.dtype), non_blocking=True)
        src_buffers = dict(self.forge.model.named_buffers())      # e.g. the routers' selection bias
        for name, b in engine.model.named_buffers():
            s = src_buffers.get(name)
            if s is not None and s.shape == b.shape:
                b.copy_(s.to(b.device, b.dtype))

    def run(self) -> dict | None:
        """Rank 0 returns the validation summaries; the other ranks return None when the leader says stop."""
        if self.rank != 0:
            follow(self.trainer, self.forge)
            return None
        try:
            return asyncio.run(self._run())
        finally:
            if isinstance(self.trainer, _LeaderTrainer):
                _announce(("stop",))

    async def _run(self) -> dict:
        out = await self.controller.run()
        await self.controller.close()
        logger.info("RL job finished")
        return out

    def close(self) -> None:
        self.forge.close()
