"""The asynchronous RL loop: rollouts are generated while the trainer trains, with bounded staleness.

Four kinds of coroutines share one event loop::

    data input  --add_work-->  [ work buffer ]  --claim_next-->  rollout workers (one per active slot)
                                     |  ^                              |
                                     |  '------- finalize_work --------'
                               take_finalized (windowed FIFO)
                                     v
                                  batcher  --TrainingBatch (queue of 1)-->  trainer loop
                                                                                |  optimizer step v -> v + 1
                         release of the trained slots  <--  generators pull v+1 <--  trainer push

* the data-input loop draws dataset samples and admits a prompt group whenever an active slot is free;
* every rollout worker claims a group, drives its ``num_samples_per_prompt`` sibling rollouts through the generator
  router, scores them and finalises the group (a failed group is finalised empty, with a failure metric);
* the batcher turns finalised groups into training samples and, once ``num_prompts_per_train_step`` trainable groups
  are present, into the packed microbatch grid of one step;
* the trainer loop runs forward / backward over the grid, steps the optimizer, and starts the weight transfer
  (trainer push, then generator pull, then release of the slots just trained) in the background: it runs under the
  next step's forward / backward and is awaited right before the weights change again.

With ``P`` prompts per step and ``S = target_offpolicy_steps`` the buffer admits ``B = (S + 1) P`` groups; the
batcher may look ``W = max(1, floor(window_fraction * B))`` groups past the oldest one, and a sample is never
trained more than ``(B + W - 2) // P`` versions after it was generated (checked at consume time).

Parity: torchtitan/experiments/rl/controller.py:156-1174, components/weight_sync.py:30-132, train.py (which
provisions Monarch meshes; ``train.py`` of this package builds the same objects in the job's own ranks).
"""

from __future__ import annotations

import asyncio
import dataclasses
import math
import time
import warnings
from dataclasses import dataclass, field
from typing import Any, Sequence

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from . import metrics as m
from .batching import Batcher, TrainingSampleBuilder
from .engine import SamplingConfig
from .policy_trainer import PolicyTrainer
from .recorder import (RolloutSampleRecorder, combine_microbatch_metrics, compute_perf_ratio_metrics,
                       compute_policy_age_metrics, compute_rollout_metrics)
from .renderer import ChatRenderer
from .rollouter import Rollouter
from .routing import InterGeneratorRouter
from .records import RolloutGroup, TrainingBatch
from .work_buffer import RolloutGroupWork, RolloutGroupWorkBuffer

__all__ = ["ValidationConfig", "AsyncLoopConfig", "WeightSyncManager", "AsyncController"]


@dataclass(kw_only=True, slots=True)
class ValidationConfig:
    num_samples: int = 20
    """Held-out prompts answered greedily (one rollout each) before and after training; 0 skips validation."""


@dataclass(kw_only=True, slots=True)
class AsyncLoopConfig(Configurable.Config):
    num_training_steps: int = 10
    num_prompts_per_train_step: int = 8
    num_samples_per_prompt: int = 8
    target_offpolicy_steps: int = 3
    window_fraction: float | None = 0.3
    """Share of the buffer the batcher may look ahead past an unfinished head; None: strict FIFO."""
    max_consecutive_untrainable_groups: int | None = 4096
    """Stop the job when this many prompt groups in a row yield nothing to train on (generation keeps failing, or
    every group's rewards are all equal and such groups are dropped: a policy that always or never succeeds gives no
    signal, and the trainer would wait forever).  None: keep waiting."""
    training_sample_builder: TrainingSampleBuilder.Config = field(default_factory=TrainingSampleBuilder.Config)
    batcher: Batcher.Config = field(default_factory=Batcher.Config)
    validation: ValidationConfig = field(default_factory=ValidationConfig)

    def __post_init__(self):
        if self.num_prompts_per_train_step < 1:
            raise ValueError(f"num_prompts_per_train_step must be >= 1, got {self.num_prompts_per_train_step}")
        if self.target_offpolicy_steps < 0:
            raise ValueError(f"target_offpolicy_steps must be >= 0, got {self.target_offpolicy_steps}")
        if self.window_fraction is not None and not 0 < self.window_fraction <= 1:
            raise ValueError(f"window_fraction must be None or in (0, 1], got {self.window_fraction}")
        if self.window_fraction is not None and self.window_fraction * self.max_active_rollout_groups < 1:
            warnings.warn(f"window_fraction={self.window_fraction} of {self.max_active_rollout_groups} groups is below "
                          "one group: strict FIFO", stacklevel=2)

    @property
    def max_active_rollout_groups(self) -> int:
        return (self.target_offpolicy_steps + 1) * self.num_prompts_per_train_step

    @property
    def window_size(self) -> int:
        if self.window_fraction is None:
            return 1
        return max(1, math.floor(self.window_fraction * self.max_active_rollout_groups))

    @property
    def max_offpolicy_steps(self) -> int:
        return (self.max_active_rollout_groups + self.window_size - 2) // self.num_prompts_per_train_step


class WeightSyncManager:
    """Trainer push -> generator pull -> release of the trained slots, as background tasks that run under the next
    step's forward / backward.  Both are awaited before the next optimizer step, which overwrites the weights the
    generators are reading."""

    def __init__(self, *, trainer: PolicyTrainer, router: InterGeneratorRouter, buffer: RolloutGroupWorkBuffer,
                 num_prompts_per_train_step: int, call_trainer=None):
        self._trainer, self._router, self._buffer, self._n = trainer, router, buffer, num_prompts_per_train_step
        self._call = call_trainer or (lambda fn, *a: asyncio.to_thread(fn, *a))
        self._push = self._pull = None
        self.last_push_s = self.last_pull_s = 0.0

    def start_async_push_pull(self, *, version: int) -> None:
        self._push = asyncio.create_task(self._do_push())
        self._pull = asyncio.create_task(self._do_pull(version, self._push))

    async def wait_prev_push(self) -> list[m.Metric]:
        if self._push is not None:
            await self._push
        return [m.Metric("timing/weight_sync/trainer_push", m.NoReduce(self.last_push_s))]

    async def wait_prev_pull(self) -> list[m.Metric]:
        if self._pull is not None:
            await self._pull
        return [m.Metric("timing/weight_sync/generator_pull", m.NoReduce(self.last_pull_s))]

    async def wait_inflight_push_pull(self) -> None:
        await self.wait_prev_push()
        await self.wait_prev_pull()

    async def _do_push(self) -> None:
        t0 = time.perf_counter()
        await self._call(self._trainer.push_model_state_dict)
        self.last_push_s = time.perf_counter() - t0

    async def _do_pull(self, version: int, push: asyncio.Task) -> None:
        await push
        t0 = time.perf_counter()
        await self._router.pull_model_state_dict(version)
        self.last_pull_s = time.perf_counter() - t0
        # only now: groups admitted into the freed slots are generated by the weights that were just trained
        await self._buffer.release_active_groups(self._n, reason="trained")


class AsyncController(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        rollouter: Rollouter.Config
        async_loop: AsyncLoopConfig = field(default_factory=AsyncLoopConfig)
        renderer: ChatRenderer.Config = field(default_factory=ChatRenderer.Config)
        sampling: SamplingConfig = field(default_factory=SamplingConfig)
        generator_router: InterGeneratorRouter.Config = field(default_factory=InterGeneratorRouter.Config)
        rollout_recorder: RolloutSampleRecorder.Config = field(default_factory=RolloutSampleRecorder.Config)
        metrics: m.MetricsProcessor.Config = field(default_factory=m.MetricsProcessor.Config)
        dump_folder: str = "outputs/rl"
        trainer_in_thread: bool = True
        """Run forward / backward and the optimizer step in a worker thread so that generation continues meanwhile.
        Must be off when a generator shares its model object with the trainer."""

    def __init__(self, config: Config, *, trainer: PolicyTrainer, generators: Sequence[Any], tokenizer,
                 dp_degree: int = 1, loggers: Sequence[Any] = (), step_callback=None):
        self.config = config
        self.trainer = trainer
        self.step_callback = step_callback
        """``step_callback(step, last_step)`` runs after every optimizer step (the job saves checkpoints there)."""
        self.renderer = config.renderer.build(tokenizer=tokenizer)
        self.rollouter: Rollouter = config.rollouter.build()
        self.router: InterGeneratorRouter = config.generator_router.build(generators=list(generators))
        self.recorder = config.rollout_recorder.build(dump_dir=config.dump_folder)
        self.metrics = config.metrics.build(dump_folder=config.dump_folder, loggers=loggers)
        self.dp_degree = dp_degree
        stops = [s for s in self.renderer.stop_sequences if s]
        self.sampling = dataclasses.replace(config.sampling, stop_sequences=[*config.sampling.stop_sequences, *stops])
        self.start_step = trainer.policy_version
        self._buffer: RolloutGroupWorkBuffer | None = None
        self._trainer_lock = asyncio.Lock()

    # -- pieces ------------------------------------------------------------------------------------------------
    async def _call_trainer(self, fn, *args):
        """One trainer call at a time (the background weight push included): a multi-rank trainer announces each call
        to its other ranks, and two announcements must not interleave."""
        async with self._trainer_lock:
            if self.config.trainer_in_thread:
                return await asyncio.to_thread(fn, *args)
            return fn(*args)

    async def validate(self, *, step: int) -> list[m.Metric]:
        n = self.config.async_loop.validation.num_samples
        if n == 0:
            return []
        t0 = time.perf_counter()
        greedy = dataclasses.replace(self.sampling, temperature=0.0, top_p=1.0, top_k=0)

        async def one(i):
            sample = await asyncio.to_thread(self.rollouter.get_validation_sample)
            try:
                return await self.rollouter.run_group_rollouts(generate_fn=self.router.generate, sample=sample, group_id=-1 - i,
                                                               group_size=1, sampling=greedy, renderer=self.renderer)
            except Exception:
                logger.exception(f"validation group {i} failed")
                return None

        groups = [g for g in await asyncio.gather(*(one(i) for i in range(n))) if g is not None]
        self.recorder.record(is_validation=True, rollout_groups=groups, step=step)
        out = compute_rollout_metrics("rollout", [r for g in groups for r in g.rollouts])
        out.append(m.Metric("group_failures", m.Sum(float(n - len(groups)))))
        out.append(m.Metric("timing/validate", m.NoReduce(time.perf_counter() - t0)))
        return out

    async def _data_input_loop(self, buffer: RolloutGroupWorkBuffer) -> None:
        gid = 0
        while await buffer.wait_for_slot():
            sample = await asyncio.to_thread(self.rollouter.get_training_sample)
            await buffer.add_work(RolloutGroupWork(group_id=gid, sample=sample))
            gid += 1

    async def _rollout_loop(self, buffer: RolloutGroupWorkBuffer) -> None:
        while (work := await buffer.claim_next()) is not None:
            try:
                group = await self.rollouter.run_group_rollouts(
                    generate_fn=self.router.generate, sample=work.sample, group_id=work.group_id,
                    group_size=self.config.async_loop.num_samples_per_prompt, sampling=self.sampling, renderer=self.renderer)
                group.metrics = compute_rollout_metrics("rollout", group.rollouts)
                self.recorder.record(is_validation=False, rollout_groups=[group], step=self.trainer.policy_version)
            except Exception:
                logger.exception(f"rollout group {work.group_id} failed; dropped")
                group = RolloutGroup(group_id=work.group_id, rollouts=[],
                                     metrics=[m.Metric("rollout/group_failures", m.Sum(1.0))])
            await buffer.finalize_work(group)

    async def _batcher_loop(self, buffer: RolloutGroupWorkBuffer, builder: TrainingSampleBuilder, batcher: Batcher,
                            queue: "asyncio.Queue[TrainingBatch | None]") -> None:
        barren = 0
        while (group := await buffer.take_finalized()) is not None:
            samples = builder.build_from_group(rollout_group=group)
            if not samples.training_samples:
                await buffer.release_active_groups(1, reason="untrainable_group")    # nothing of it will be trained
                barren += 1
                limit = self.config.async_loop.max_consecutive_untrainable_groups
                if limit is not None and barren >= limit:
                    raise RuntimeError(f"{barren} prompt groups in a row gave nothing to train on; stopping")
                if barren % 32 == 0:
                    logger.warning(f"{barren} prompt groups in a row gave nothing to train on (failed, empty, or all "
                                   "rewards equal with drop_zero_std_reward_groups): the trainer is waiting")
            else:
                barren = 0
            batch = await asyncio.to_thread(batcher.add_training_samples, training_sample_group=samples)
            if batch is not None:
                await queue.put(batch)
        await queue.put(None)

    async def _trainer_loop(self, queue: "asyncio.Queue[TrainingBatch | None]", sync: WeightSyncManager) -> None:
        loop_cfg = self.config.async_loop
        for step in range(self.start_step + 1, loop_cfg.num_training_steps + 1):
            timer = m.MetricsTimer()
            with timer.record("timing/step/total"):
                with timer.record("timing/step/wait_for_training_batch"):
                    batch = await queue.get()
                if batch is None:
                    logger.info("batcher closed: training stops")
                    break
                age = compute_policy_age_metrics(trainer_policy_version=self.trainer.policy_version,
                                                 min_policy_versions=batch.min_policy_versions,
                                                 max_offpolicy_steps=loop_cfg.max_offpolicy_steps)
                with timer.record("timing/step/forward_backward"):
                    per_mb = [await self._call_trainer(self.trainer.forward_backward, row, batch.num_global_valid_tokens)
                              for row in batch.microbatches]
                    fb = combine_microbatch_metrics(per_mb)
                if not math.isfinite(fb["loss/mean"]):
                    raise FloatingPointError(f"step {step}: the policy loss is not finite")
                # the generators copy from the trainer's live weights (there is no staging store in between), so the
                # previous push AND pull must be over before the optimizer overwrites them; both overlapped with this
                # step's forward / backward
                with timer.record("timing/step/blocking_trainer_push"):
                    push = await sync.wait_prev_push()
                with timer.record("timing/step/blocking_generator_pull"):
                    pull = await sync.wait_prev_pull()
                with timer.record("timing/step/optim"):
                    opt = await self._call_trainer(self.trainer.optim_step)
                sync.start_async_push_pull(version=opt.policy_version)
            times = timer.flush()
            self.metrics.log(step=step, metrics=[
                *batch.metrics, *[m.Metric(k, m.NoReduce(v)) for k, v in fb.items()],
                *[m.Metric(k, m.NoReduce(v)) for k, v in opt.metrics.items()], *self._buffer.metrics(), *times, *age,
                *push, *pull, *compute_perf_ratio_metrics(num_global_valid_tokens=batch.num_global_valid_tokens,
                                                          time_metrics=times)])
            if self.step_callback is not None:
                await self._call_trainer(self.step_callback, step, step == loop_cfg.num_training_steps)
        await sync.wait_inflight_push_pull()

    # -- the whole run ------------------------------------------------------------------------------------------
    async def run(self) -> dict[str, dict[str, float]]:
        """Validation, ``num_training_steps`` optimizer steps, validation.  Returns the two validation summaries."""
        lc = self.config.async_loop
        pre = self.metrics.log(step=self.start_step, metrics=await self.validate(step=self.start_step), is_validation=True)
        self._buffer = buffer = RolloutGroupWorkBuffer(max_active_rollout_groups=lc.max_active_rollout_groups,
                                                       window_size=lc.window_size)
        logger.info(f"async RL: {lc.max_active_rollout_groups} active groups, window {lc.window_size}, "
                    f"policy age <= {lc.max_offpolicy_steps}")
        sync = WeightSyncManager(trainer=self.trainer, router=self.router, buffer=buffer,
                                 num_prompts_per_train_step=lc.num_prompts_per_train_step, call_trainer=self._call_trainer)
        batcher = lc.batcher.build(num_prompts_per_train_step=lc.num_prompts_per_train_step, dp_degree=self.dp_degree,
                                   pad_id=self.renderer.eos_token_id)
        queue: asyncio.Queue = asyncio.Queue(maxsize=1)
        background = [asyncio.create_task(self._data_input_loop(buffer), name="data_input"),
                      *[asyncio.create_task(self._rollout_loop(buffer), name=f"rollout_worker_{i}")
                        for i in range(lc.max_active_rollout_groups)],
                      asyncio.create_task(self._batcher_loop(buffer, lc.training_sample_builder.build(), batcher, queue),
                                          name="batcher")]
        trainer_task = asyncio.create_task(self._trainer_loop(queue, sync), name="trainer")
        try:
            done, _ = await asyncio.wait([trainer_task, *background], return_when=asyncio.FIRST_COMPLETED)
            for t in done:                      # only the trainer loop is finite: anything else ending is a failure
                if t is not trainer_task:
                    await t
                    raise RuntimeError(f"{t.get_name()} ended unexpectedly")
            await trainer_task
        finally:
            await buffer.close()
            for t in (*background, trainer_task):
                t.cancel()
            await asyncio.gather(*background, trainer_task, return_exceptions=True)
        post = self.metrics.log(step=lc.num_training_steps, metrics=await self.validate(step=lc.num_training_steps),
                                is_validation=True)
        for k in sorted(k for k in set(pre) | set(post) if "reward" in k):
            logger.info(f"validation {k}: {pre.get(k, float('nan')):+.3f} -> {post.get(k, float('nan')):+.3f}")
        return {"pre": pre, "post": post}

    async def close(self) -> None:
        await self.router.close_generators()
