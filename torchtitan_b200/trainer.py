"""The training loop.

``Trainer.Config`` is the root of the job configuration (sections mirror
torchtitan/trainer.py:69-116 plus ``model`` and ``kernels``).  ``Trainer`` builds
everything from it, ``train()`` runs optimizer steps:

    for each microbatch of the step: H2D copy -> forward -> fused lm_head+CE -> backward
        (per-unit gradient reduction overlaps with the rest of backward)
    global grad norm + clip scale (device scalars) -> sharded AdamW (+ weight refresh)
    -> LR schedule -> metrics on logging steps (the only routine host sync)

Losses are divided by the global number of valid tokens of the whole step, so no
gradient averaging happens anywhere (parity: trainer.py:842-1008).
"""

from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch
import torch.distributed as dist

from torchtitan_b200.components.data import BaseDataLoader, DataloaderExhaustedError
from torchtitan_b200.components.loss import IGNORE_INDEX, BaseLoss, CrossEntropyLoss, LinearCrossEntropyLoss
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import MoEBiasUpdater, OptimizersContainer, clip_grad_norm_
from torchtitan_b200.config import (
    ActivationCheckpointConfig, CommConfig, CompileConfig, Configurable, DebugConfig, KernelConfig,
    ModelSelectConfig, OverrideConfig, ParallelismConfig, TrainingConfig, apply_overrides,
)
from torchtitan_b200.models import ModelSpec, get_model_spec
from torchtitan_b200.ops import functional as OF
from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.parallel.parallel_dims import ParallelDims
from torchtitan_b200.utils import structured_logger as sl
from torchtitan_b200.utils.device import GarbageCollection, device_name, get_local_device, get_peak_flops
from torchtitan_b200.utils.logging import logger

__all__ = ["Trainer"]


@dataclass(kw_only=True, slots=True)
class LossConfig:
    name: str = "linear_cross_entropy"
    """``linear_cross_entropy`` (chunked fused lm_head + CE) | ``cross_entropy`` | ``mse``."""
    num_chunks: int = 8


class Trainer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        model_spec: Any = None
        model: ModelSelectConfig = field(default_factory=ModelSelectConfig)
        hf_assets_path: str = "./tests/assets/tokenizer"
        dump_folder: str = "./outputs"
        profiler: Any = None
        metrics: MetricsProcessor.Config = field(default_factory=MetricsProcessor.Config)
        tokenizer: Any = None
        dataloader: BaseDataLoader.Config = field(default_factory=BaseDataLoader.Config)
        optimizer: OptimizersContainer.Config = field(default_factory=OptimizersContainer.Config)
        lr_scheduler: LRSchedulersContainer.Config = field(default_factory=LRSchedulersContainer.Config)
        training: TrainingConfig = field(default_factory=TrainingConfig)
        parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
        checkpoint: Any = None
        activation_checkpoint: ActivationCheckpointConfig = field(default_factory=ActivationCheckpointConfig)
        compile: CompileConfig = field(default_factory=CompileConfig)
        comm: CommConfig = field(default_factory=CommConfig)
        validator: Any = None
        debug: DebugConfig = field(default_factory=DebugConfig)
        override: OverrideConfig = field(default_factory=OverrideConfig)
        loss: LossConfig = field(default_factory=LossConfig)
        kernels: KernelConfig = field(default_factory=KernelConfig)

        def __post_init__(self):
            from torchtitan_b200.components.checkpoint import CheckpointManager
            from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer
            from torchtitan_b200.components.validate import Validator
            from torchtitan_b200.utils.profiler import Profiler

            if self.profiler is None:
                self.profiler = Profiler.Config()
            if self.checkpoint is None:
                self.checkpoint = CheckpointManager.Config()
            if self.validator is None:
                self.validator = Validator.Config()
            if self.tokenizer is None:
                self.tokenizer = HuggingFaceTokenizer.Config()

        def validate(self) -> None:
            """Cross-field checks (parity: trainer.py:118-199)."""
            t, p = self.training, self.parallelism
            if t.num_tokens_per_microbatch_per_dp_rank <= 0:
                raise ValueError("training.num_tokens_per_microbatch_per_dp_rank must be positive")
            if t.max_context_length <= 0:
                raise ValueError("training.max_context_length must be positive")
            if p.pipeline_parallel_degree > 1 and p.num_pp_microbatches < 1:
                raise ValueError("parallelism.num_pp_microbatches must be >= 1")
            if self.compile.passes:
                from torchtitan_b200.experiments.graph_trainer import apply_passes

                logger.info(f"compile.passes: {apply_passes(self, list(self.compile.passes), run_precompile=False)}")
            if self.compile.enable:
                logger.warning("compile.enable is accepted for compatibility; this framework runs hand-written "
                               "kernels and CUDA graphs instead of a tracing compiler")
            if self.compile.enable_async_tensor_parallel and p.tensor_parallel_degree > 1 and p.tp_comm == "nccl":
                # the reference's async TP overlaps the all-gather / reduce-scatter with the GEMM through the compiler
                # (distributed/tensor_parallel.py:19-95); here it selects the GEMM kernels with the collective inside
                if not p.enable_sequence_parallel:
                    raise ValueError("async tensor parallelism needs sequence parallelism")
                p.tp_comm = "nvlink"
                logger.info("compile.enable_async_tensor_parallel: tensor-parallel collectives run inside the GEMM "
                            "kernels (parallelism.tp_comm = nvlink)")
            if not t.disable_cuda_graphs and p.pipeline_parallel_degree > 1:
                raise ValueError("CUDA graphs cannot be combined with pipeline parallelism")
            if self.checkpoint is not None and self.checkpoint.enable and self.checkpoint.keep_latest_k == 1:
                raise ValueError("checkpoint.keep_latest_k must be 0 (keep all) or >= 2")

        def to_json(self) -> str:
            d = self.to_dict()
            d.pop("model_spec", None)
            return json.dumps(d, indent=2, default=str)

    # ------------------------------------------------------------------
    def __init__(self, config: "Trainer.Config", **_):
        self.config = config
        c = config
        config.validate()
        from torchtitan_b200.parallel.symm import status_monitor

        status_monitor.clear()   # arenas of an earlier trainer in this process are gone
        if c.parallelism.ep_overflow == "drop":
            status_monitor.tolerated |= 8
        self.device = get_local_device()
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if c.debug.batch_invariant:
            pinned = dist_utils.pin_nccl_for_batch_invariance()
            logger.info(f"batch-invariant mode: NCCL pinned with {pinned}")
        with sl.span("torch_distributed_init"):
            world = dist_utils.init_distributed(c.comm, self.device, dump_folder=c.dump_folder,
                                                enable_cpu_backend=c.training.enable_cpu_offload)
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.pdims = ParallelDims.from_config(c.parallelism, world, rank).build()
        pd = self.pdims
        if "precompile" in c.compile.passes:       # rank 0 builds the extension, the others wait and load it
            from torchtitan_b200.experiments.graph_trainer import precompile

            precompile()
        div = pd.seq_len_divisor
        if c.training.num_tokens_per_microbatch_per_dp_rank % div:
            raise ValueError(f"tokens per microbatch ({c.training.num_tokens_per_microbatch_per_dp_rank}) must be "
                             f"divisible by tp * 2cp = {div}")
        if c.debug.print_config and rank == 0:
            logger.info(f"Running with config:\n{c.to_json()}")
        if c.debug.save_config_file and rank == 0:
            os.makedirs(c.dump_folder, exist_ok=True)
            with open(os.path.join(c.dump_folder, c.debug.save_config_file), "w") as f:
                f.write(c.to_json())
        self.gc_handler = GarbageCollection(c.training.gc_freq, c.training.gc_debug)
        self.seed = dist_utils.set_determinism(pd, self.device, c.debug.seed, c.debug.deterministic,
                                               c.debug.deterministic_warn_only)
        OF.settings.gemm = c.kernels.gemm
        OF.settings.attention = c.kernels.attention
        OF.settings.strict_native = False
        if c.debug.batch_invariant:
            from torchtitan_b200.experiments.rl.batch_invariance import enable_batch_invariant_mode

            enable_batch_invariant_mode(True)

        # ---- model ------------------------------------------------------
        spec: ModelSpec = c.model_spec or get_model_spec(c.model.name, c.model.flavor)
        self.model_spec = spec
        model_cfg = spec.model
        model_cfg.update_from_config(trainer_config=c)
        from torchtitan_b200.components.quantization import apply_converters

        apply_converters(model_cfg, c.model.converters, c)
        if c.override.imports:
            done = apply_overrides(model_cfg, c.override.imports)
            logger.info(f"applied overrides: {done}")
        if c.debug.moe_force_load_balance:
            for ref in model_cfg.walk(object, descend_into_matches=True):
                if hasattr(ref.config, "_debug_force_load_balance"):
                    ref.config._debug_force_load_balance = True
        self.model_config = model_cfg
        dtype = torch.float32 if c.training.dtype == "float32" else torch.bfloat16
        self.metrics_processor: MetricsProcessor = c.metrics.build(
            pdims=pd, device=self.device, dump_folder=c.dump_folder, job_config_dict=c.to_dict())
        self.loss_fn = self._build_loss()

        # ---- gradient accumulation ---------------------------------------
        tok_mb = c.training.num_tokens_per_microbatch_per_dp_rank
        per_pass = tok_mb * pd.dp_degree * (c.parallelism.num_pp_microbatches if pd.pp_enabled else 1)
        step_tokens = c.training.num_tokens_per_train_step
        if step_tokens == -1:
            step_tokens = per_pass
        if step_tokens % per_pass:
            raise ValueError(f"training.num_tokens_per_train_step ({step_tokens}) must be a multiple of "
                             f"tokens_per_microbatch * dp degree (* pp microbatches) = {per_pass}")
        self.gradient_accumulation_steps = step_tokens // per_pass
        self.tokens_per_step_per_dp_rank = step_tokens // pd.dp_degree

        # ---- parallelise + materialise --------------------------------------
        with sl.span("model_parallelism_init"):
            with torch.device("meta"):
                prev = torch.get_default_dtype()
                torch.set_default_dtype(dtype)
                try:
                    model = model_cfg.build()
                finally:
                    torch.set_default_dtype(prev)
            self.pp_schedule = None
            if pd.pp_enabled:
                if spec.pipelining_fn is None:
                    raise ValueError(f"model {spec.name} does not support pipeline parallelism")
                (self.pp_schedule, self.model_parts, self.engines, self.pp_has_first_stage,
                 self.pp_has_last_stage) = spec.pipelining_fn(
                    model, pdims=pd, job_config=c, device=self.device, seed=self.seed,
                    parallelize_fn=spec.parallelize_fn, loss_fn=self.loss_fn,
                    grad_accum_steps=self.gradient_accumulation_steps)
            else:
                engine = spec.parallelize_fn(model, pdims=pd, job_config=c, device=self.device, seed=self.seed,
                                             grad_accum_steps=self.gradient_accumulation_steps)
                self.model_parts = [model]
                self.engines = [engine]
                if isinstance(self.loss_fn, LinearCrossEntropyLoss):
                    self.loss_fn.set_lm_head(model.lm_head, tp=model.tp,
                                             softcap=getattr(model_cfg, "final_logit_softcap", None),
                                             multiplier=getattr(model_cfg, "final_logit_multiplier", 1.0))
                if getattr(model, "mtp_layers", None) is not None:
                    # multi-token prediction: the same loss on every depth's output, weighted
                    from torchtitan_b200.models.deepseek_v3.mtp import MTPLoss

                    self.loss_fn = MTPLoss(self.loss_fn, mtp_scale=getattr(model_cfg, "mtp_scale", 0.3))
        self.model = self.model_parts[0]

        nparams, flops = model_cfg.get_nparams_and_flops(None, c.training.max_context_length)
        self.metrics_processor.num_flops_per_token = flops
        self.metrics_processor.gpu_peak_flops = get_peak_flops(device_name(self.device))
        self.metrics_processor.quantized = bool(c.model.converters and any(
            k in ("mxfp8", "float8", "nvfp4") for k in c.model.converters))
        logger.info(f"Model {spec.name} {spec.flavor} size: {nparams:,} total parameters, "
                    f"{flops:.3e} FLOPs/token")

        # ---- optimizer, schedule, data, checkpoints ---------------------------
        self.optimizers: OptimizersContainer = c.optimizer.build(engines=self.engines)
        full_ac = c.activation_checkpoint.mode == "full"
        bias_updater = MoEBiasUpdater(self.model_parts, pd, full_ac=full_ac)
        if bias_updater.moes:
            self.optimizers.register_step_pre_hook(bias_updater)
        if spec.post_optimizer_build_fn is not None:
            spec.post_optimizer_build_fn(self.optimizers, self.model_parts, pd)
        self.lr_schedulers: LRSchedulersContainer = c.lr_scheduler.build(
            optimizers=self.optimizers, training_steps=c.training.steps)
        self.tokenizer = None
        if c.dataloader.dataset not in ("synthetic", "synthetic_mm"):
            self.tokenizer = c.tokenizer.build(tokenizer_path=c.hf_assets_path)
        mm_kw = {}
        vis = getattr(model_cfg, "vision_encoder", None)
        if vis is not None:     # the collator patchifies for this tower
            mm_kw = dict(patch_size=vis.patch_size, spatial_merge=vis.spatial_merge, in_channels=vis.in_channels,
                         image_token_id=model_cfg.image_token_id)
        self.dataloader = c.dataloader.build(
            dp_world_size=pd.dp_degree, dp_rank=pd.dp_rank, num_tokens_per_batch=tok_mb,
            max_context_length=c.training.max_context_length, vocab_size=model_cfg.vocab_size,
            tokenizer=self.tokenizer, **mm_kw)
        self.step = 0
        self.ntokens_seen = 0
        self.checkpointer = c.checkpoint.build(
            trainer=self, dump_folder=c.dump_folder, pdims=pd)
        self.validator = None
        if c.validator.enable:
            self.validator = c.validator.build(trainer=self)
        self.profiler_config = c.profiler
        self._graph_runner = None
        self._mb_index = 0
        if (not c.training.disable_cuda_graphs and self.device.type == "cuda" and not pd.pp_enabled
                and not c.activation_checkpoint.cpu_offload   # host copies cannot be captured
                # the all-to-all dispatcher and the exact mode of the NVLink dispatcher read row counts on the host
                and not (pd.ep_enabled and (c.parallelism.ep_comm == "nccl" or not c.parallelism.ep_capacity_factor))):
            from torchtitan_b200.parallel.cudagraph import CUDAGraphRunner

            eng = self.engines[0]
            self._graph_runner = CUDAGraphRunner(
                self._fwd_bwd_tensors,
                snapshot=lambda: [u.grad_shard_valid for u in eng.units],
                after_replay=lambda st: [setattr(u, "grad_shard_valid", v) for u, v in zip(eng.units, st)])
        self._inv_tokens_cache = None
        logger.info(
            f"Trainer ready: tokens/microbatch/dp-rank {tok_mb}, grad accumulation {self.gradient_accumulation_steps}, "
            f"steps {c.training.steps}, warmup {c.lr_scheduler.warmup_steps}, mesh "
            f"pp{pd.pp} dp_rep{pd.dp_replicate} dp_shard{pd.dp_shard} cp{pd.cp} tp{pd.tp} ep{pd.ep}")

    # ------------------------------------------------------------------
    def _build_loss(self) -> BaseLoss:
        lc = self.config.loss
        if lc.name == "linear_cross_entropy":
            return LinearCrossEntropyLoss(LinearCrossEntropyLoss.Config(num_chunks=lc.num_chunks))
        if lc.name == "cross_entropy":
            return CrossEntropyLoss(CrossEntropyLoss.Config())
        if lc.name == "mse":
            from torchtitan_b200.components.loss import MSELoss

            return MSELoss()
        raise ValueError(f"unknown loss '{lc.name}'")

    # ------------------------------------------------------------------
    def batch_generator(self, data_iterable) -> Iterator:
        it = iter(data_iterable)
        while True:
            t0 = time.perf_counter()
            try:
                with sl.span("fetching_batch"):
                    batch = next(it)
            except StopIteration as e:
                raise DataloaderExhaustedError() from e
            self.metrics_processor.data_loading_times.append(time.perf_counter() - t0)
            yield batch

    def post_dataloading_process(self, inputs: dict[str, torch.Tensor], labels: torch.Tensor):
        """H2D copy, context-parallel sharding, attention context."""
        dev = self.device
        tokens = inputs["input"].to(dev, non_blocking=True)
        positions = inputs["positions"].to(dev, non_blocking=True)
        labels = labels.to(dev, non_blocking=True)
        q_pos = None
        model = self.model
        # anything else in the batch (image patches, grids) goes to the model as keyword arguments
        self._extra_inputs = {k: (v.to(dev, non_blocking=True) if k != "grid_hw" else v)
                              for k, v in inputs.items() if k not in ("input", "positions")}
        if self.pdims.cp_enabled:
            if self._extra_inputs:
                raise NotImplementedError("multimodal batches are not supported with context parallelism")
            from torchtitan_b200.parallel.context_parallel import ptrr_assignment, shard_for_cp

            if model.cp.load_balancer == "ptrr":
                # the balancer is built from this batch's documents (host copy of the positions; same on every cp rank)
                host_pos = inputs["positions"] if not inputs["positions"].is_cuda else inputs["positions"].cpu()
                model.cp.assignment = ptrr_assignment(host_pos, model.cp.size)
            tokens, positions, labels, q_pos = shard_for_cp(model.cp, tokens, positions, labels)
        return tokens, positions, labels, q_pos

    def forward_backward_step(self, inputs, labels, global_valid: torch.Tensor) -> torch.Tensor:
        with sl.span("post_dataloading_process"):
            tokens, positions, labels, q_pos = self.post_dataloading_process(inputs, labels)
        if self.pdims.pp_enabled:
            return self.pp_forward_backward_step(tokens, positions, labels, q_pos, global_valid)
        if self._graph_runner is not None and q_pos is None and not self._extra_inputs:
            self.engines[0].wait_optimizer()   # a replayed graph has no per-unit waits on the previous optimizer step
            key = (min(self._mb_index, 1), tuple(tokens.shape))
            self._mb_index += 1
            with sl.span("fwd_bwd"):
                return self._graph_runner(key, tokens, positions, labels, global_valid).detach()
        return self._fwd_bwd_tensors(tokens, positions, labels, global_valid, q_pos)

    def _fwd_bwd_tensors(self, tokens, positions, labels, global_valid, q_pos=None) -> torch.Tensor:
        model = self.model
        ac = self.config.activation_checkpoint
        if ac.cpu_offload:
            from torchtitan_b200.parallel.activation_offload import offload_activations

            offload = offload_activations(min_bytes=ac.cpu_offload_min_bytes)
        else:
            import contextlib

            offload = contextlib.nullcontext()
        with sl.span("fwd_bwd"), offload:
            ctx = model.build_context(positions, q_pos)
            extra = getattr(self, "_extra_inputs", None) or {}
            if self.loss_fn.needs_hidden:
                pred = model(tokens, positions, ctx, return_hidden=True, **extra)
            else:
                pred = model(tokens, positions, ctx, **extra)
            if getattr(self.loss_fn, "needs_positions", False):
                loss = self.loss_fn(pred, labels, global_valid, positions=positions)
            else:
                loss = self.loss_fn(pred, labels, global_valid)
            del pred
            loss.backward()
            self.engines[0].finish_backward()
        return loss.detach()

    def pp_forward_backward_step(self, tokens, positions, labels, q_pos, global_valid) -> torch.Tensor:
        from torchtitan_b200.parallel.pipeline import run_pipeline_step

        return run_pipeline_step(self, tokens, positions, labels, q_pos, global_valid)

    def train_step(self, data_iterator) -> None:
        c = self.config
        pd = self.pdims
        self.optimizers.zero_grad()
        self._mb_index = 0
        n_mb = self.gradient_accumulation_steps * (c.parallelism.num_pp_microbatches if pd.pp_enabled else 1)
        microbatches = []
        host_valid = 0
        dev_valid = None
        for _ in range(n_mb):
            inputs, labels = next(data_iterator)
            if labels.is_cuda:  # device-resident batches: count without a host sync
                n = (labels != IGNORE_INDEX).sum().to(torch.float32)
                dev_valid = n if dev_valid is None else dev_valid + n
            else:
                host_valid += int((labels != IGNORE_INDEX).sum())
            microbatches.append((inputs, labels))
            self.ntokens_seen += labels.numel() * pd.dp_degree
            self.metrics_processor.ntokens_since_last_log += labels.numel()
        valid = torch.tensor([float(host_valid)], dtype=torch.float32).to(self.device, non_blocking=True)
        if dev_valid is not None:
            valid = valid + dev_valid
        g = pd.group("batch")
        if g is not None:
            dist.all_reduce(valid, group=g)

        losses = []
        if pd.pp_enabled:
            per = c.parallelism.num_pp_microbatches
            for a in range(self.gradient_accumulation_steps):
                group = microbatches[a * per:(a + 1) * per]
                inputs = {k: torch.stack([m[0][k] for m in group]) for k in group[0][0]}
                labels = torch.stack([m[1] for m in group])
                losses.append(self.forward_backward_step(inputs, labels, valid))
        else:
            for inputs, labels in microbatches:
                losses.append(self.forward_backward_step(inputs, labels, valid))
        loss = torch.stack([l.reshape(()) for l in losses]).sum()
        loss_finite = torch.isfinite(loss)

        grad_norm = clip_grad_norm_(self.engines, c.training.max_norm, pd, loss_finite=loss_finite,
                                    optimizers=self.optimizers)
        self.checkpointer.maybe_wait_for_staging()
        with sl.span("optim"):
            self.optimizers.step()
            self.lr_schedulers.step()
        self._last_loss, self._last_grad_norm = loss, grad_norm
        self._poll_device_status(sync=False)

        if not self.metrics_processor.should_log(self.step):
            return
        self._poll_device_status(sync=True)
        with sl.span("collect_dist_metrics"):
            lg = pd.group("loss")
            stats = torch.stack([loss.float().reshape(()), grad_norm.float().reshape(())])
            if pd.pp_enabled:
                # only the last stage knows the loss
                dist.all_reduce(stats[:1], group=pd.group("pp"))
            total = stats[0].clone()
            mx = stats[0].clone()
            if lg is not None:
                dist.all_reduce(total, group=lg)
                dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=lg)
            vals = torch.stack([total, mx, stats[1]]).cpu().tolist()  # the routine host sync
        global_avg, global_max, gn = vals
        if not (global_avg == global_avg and abs(global_avg) != float("inf") and gn == gn and abs(gn) != float("inf")):
            raise RuntimeError(
                f"non-finite loss ({global_avg}) or gradient norm ({gn}) at step {self.step}: the optimizer "
                "update of this step was skipped on the device")
        extra = {"n_tokens_seen": self.ntokens_seen}
        extra.update(self.lr_schedulers.get_metrics())
        self.metrics_processor.log(self.step, global_avg, global_max, gn, extra_metrics=extra)

    def _poll_device_status(self, sync: bool) -> None:
        """Raise when a bounded device-side wait of an NVLink path or of a kernel pipeline expired.

        Every step queues an asynchronous copy of the arenas' status words and examines the copy of
        the step before (no stall); logging steps, which synchronise anyway, read the current
        values of the arenas and of the kernels' own status words."""
        from torchtitan_b200.parallel.symm import status_monitor

        if not sync:
            status_monitor.poll()
            return
        status_monitor.check()
        from torchtitan_b200.ops import ext

        if self.device.type == "cuda" and ext.available():
            ops = ext.require()
            bits = int(ops.status(True)) | int(ops.gemm_status(True)) | int(ops.flash_status(True))
            if bits & 4:
                raise RuntimeError(f"a bounded wait inside a kernel pipeline expired (status {bits:#x}): results of this "
                                   "step are incomplete")

    # ------------------------------------------------------------------
    def train(self) -> None:
        c = self.config
        self.checkpointer.load(step=c.checkpoint.load_step)
        logger.info(f"Training starts at step {self.step + 1}")
        from torchtitan_b200.utils.profiler import Profiler

        data_iterator = self.batch_generator(self.dataloader)
        with Profiler(self.profiler_config, global_step=self.step, base_folder=c.dump_folder,
                      rank=self.pdims.rank) as prof:
            while self.step < c.training.steps:
                self.step += 1
                sl.set_step(self.step)
                if self.gc_handler.run(self.step):
                    sl.add_step_tag("gc")
                try:
                    with sl.span("step"):
                        self.train_step(data_iterator)
                except DataloaderExhaustedError:
                    logger.warning("Ran out of data; last step was canceled.")
                    self.step -= 1
                    break
                self.checkpointer.save(self.step, last_step=(self.step == c.training.steps))
                if self.validator is not None and self.validator.should_validate(self.step):
                    with sl.span("eval"):
                        self.validator.validate(self.model_parts, self.step)
                prof.step()
                if self.step == 1:
                    dist_utils.set_pg_timeouts(c.comm.train_timeout_seconds, self.pdims)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        logger.info("Training completed")

    # ------------------------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        return {"step": self.step, "ntokens_seen": self.ntokens_seen}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.step = int(sd["step"])
        self.ntokens_seen = int(sd.get("ntokens_seen", 0))

    def close(self) -> None:
        if getattr(self, "checkpointer", None) is not None:
            self.checkpointer.close()
        if getattr(self, "metrics_processor", None) is not None:
            self.metrics_processor.close()
