"""Headline benchmark: Llama-3.1-8B pre-training throughput (tokens/s), FSDP, bf16, seq 8192,
local batch 1, synthetic uniform tokens, random init -- the config of the reference's published
B200 numbers (torchtitan/components/quantization/mxfp8.md:157-161).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Two measurements of the same metric are reported on one JSON line:

* ``value``: K optimizer steps timed on the device with CUDA events between a barrier +
  synchronize on both sides, inputs already resident on the GPU; max over ranks.
* ``e2e.value``: K steps through the public ``Trainer.train_step`` API, each step fetching its
  batch from pinned host memory (host->device copy inside the timed region) and reading the loss
  back to the host.

Every step does the full work: forward, backward, gradient reduction, grad-norm clipping and
the AdamW update.  The per-step working set (tens of GB) is far larger than the 126 MB L2, so
no explicit L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_SEC_PER_GPU = 8307.5  # Llama3-8B bf16, 8x B200, FSDP2 + compile (reference's published number)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=["native", "reference"])
    p.add_argument("--model", default=None)           # explicit values win over the preset's
    p.add_argument("--flavor", default=None)
    p.add_argument("--seq-len", type=int, default=None)
    p.add_argument("--local-batch", type=int, default=None)
    p.add_argument("--fsdp-comm", default=os.environ.get("TB200_FSDP_COMM", "auto"))
    p.add_argument("--gemm", default=os.environ.get("TB200_GEMM", "tcgen05"))
    p.add_argument("--attention", default=os.environ.get("TB200_ATTENTION", "native"))
    p.add_argument("--opt-state", default=None, choices=["fp32", "bf16"])
    p.add_argument("--ac", default=None)
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--converters", default=None, help="comma-separated model converters, e.g. mxfp8 (a separate, "
                   "lower-precision measurement: the headline stays bf16)")
    p.add_argument("--preset", default="fsdp", choices=sorted(PRESETS),
                   help="fsdp = the headline (Llama-3 8B, FSDP over all ranks); the others are the multi-dimensional "
                        "configurations listed in PRESETS")
    p.add_argument("--comm", default="default", choices=["default", "nvlink", "nccl"],
                   help="nvlink / nccl switch every collective path of the preset together (FSDP, TP, CP, EP) between the "
                        "in-kernel NVLink transport and the NCCL arm; default keeps each path's default")
    p.add_argument("--reshard", default=None, choices=["default", "always", "never"],
                   help="parallelism.fsdp_reshard_after_forward")
    p.add_argument("--par", action="append", default=[], metavar="KEY=VALUE",
                   help="override one field of the parallelism section (repeatable), e.g. --par tensor_parallel_degree=1")
    return p.parse_args()


# Multi-dimensional benchmark configurations (8 GPUs unless noted).  Each entry: model, flavor, sequence length,
# sequences per microbatch, parallelism overrides, converters, optimizer state dtype, activation checkpointing.
PRESETS = {
    "fsdp": {},
    # Llama-3.1 8B, FSDP x async TP 2 x CP 2, 32k tokens, MXFP8 linears
    "3d_mxfp8_32k": dict(model="llama3", flavor="8B", seq_len=32768, local_batch=1, converters="mxfp8", ac="selective",
                         par=dict(tensor_parallel_degree=2, context_parallel_degree=2)),
    # Qwen3-30B-A3B-shaped MoE, expert parallel over all ranks, FSDP on the rest.  A random-init router sends most
    # tokens to a few experts (one rank can receive several times the balanced load), so throughput runs assign
    # experts round-robin (debug.moe_force_load_balance, as the reference does for its throughput runs): the same
    # rows and FLOPs per step on both arms, and the static receive buffers of the NVLink dispatcher fit.
    "moe_ep8": dict(model="qwen3", flavor="30B-A3B", seq_len=4096, local_batch=2, ac="selective", force_balance=True,
                    par=dict(expert_parallel_degree=-1, ep_capacity_factor=1.25)),
    # Llama-3.1 70B, PP 2 (interleaved 1F1B, two virtual stages per rank) x TP 2 x FSDP, bf16 optimizer states, full AC
    "70b_pp2tp2": dict(model="llama3", flavor="70B", seq_len=8192, local_batch=1, opt_state="bf16", ac="full",
                       par=dict(pipeline_parallel_degree=2, tensor_parallel_degree=2,
                                pipeline_parallel_schedule="Interleaved1F1B", pipeline_parallel_layers_per_stage=21,
                                num_pp_microbatches=8)),
}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period: float = 0.2):
        self.index, self.period = index, period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def reference_arm(args) -> None:
    """Run the unmodified upstream torchtitan through its own Trainer (see baseline/reference_arm.py)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("tb200_reference_arm", os.path.join(ROOT, "baseline", "reference_arm.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if ROOT in sys.path:
        sys.path.remove(ROOT)  # nothing of this repo's package is importable on the reference path
    if args.preset != "fsdp":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm covers the FSDP headline only; the image's "
                              "torchtitan 0.1.0 has no counterpart wired for preset " + args.preset}), flush=True)
        return
    mod.run(args, ROOT, ClockSampler)


def apply_preset(args) -> dict:
    """Fold the preset into ``args``; returns the parallelism overrides."""
    pre = PRESETS[args.preset]
    base = dict(model="llama3", flavor="8B", seq_len=8192, local_batch=1, opt_state="fp32", ac="selective")
    for key, default in base.items():
        if getattr(args, key) is None:
            setattr(args, key, pre.get(key, default))
    if args.converters is None:
        args.converters = pre.get("converters", "")
    par = dict(pre.get("par", {}))
    if par.get("expert_parallel_degree") == -1:
        par["expert_parallel_degree"] = args.gpus
    if args.comm != "default":
        par.update(fsdp_comm=args.comm, tp_comm=args.comm, cp_transport=args.comm, ep_comm=args.comm)
    else:
        par.setdefault("fsdp_comm", args.fsdp_comm)
    if args.reshard is not None:
        par["fsdp_reshard_after_forward"] = args.reshard
    for item in args.par:
        key, _, val = item.partition("=")
        try:
            par[key] = int(val)
        except ValueError:
            try:
                par[key] = float(val)
            except ValueError:
                par[key] = val
    return par


def main() -> None:
    args = parse_args()
    par_overrides = apply_preset(args)
    if args.impl == "reference":
        reference_arm(args)
        return
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
    import torch
    import torch.distributed as dist

    from torchtitan_b200.components.checkpoint import CheckpointManager
    from torchtitan_b200.components.data import BaseDataLoader
    from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
    from torchtitan_b200.components.metrics import MetricsProcessor
    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.config import ActivationCheckpointConfig, KernelConfig, ModelSelectConfig, ParallelismConfig, TrainingConfig
    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.trainer import Trainer
    from torchtitan_b200.utils.logging import init_logger

    init_logger()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    T = args.seq_len * args.local_batch
    steps_total = args.warmup * 2 + args.steps * 2 + 4
    cfg = Trainer.Config(
        model=ModelSelectConfig(name=args.model, flavor=args.flavor),
        dump_folder="/tmp/tb200_bench",
        metrics=MetricsProcessor.Config(log_freq=10 ** 9),
        dataloader=BaseDataLoader.Config(dataset="synthetic", seed=0),
        optimizer=OptimizersContainer.Config(lr=3e-4, implementation="fused" if args.opt_state == "fp32" else "fused_opt_states_bf16"),
        lr_scheduler=LRSchedulersContainer.Config(warmup_steps=2),
        training=TrainingConfig(num_tokens_per_microbatch_per_dp_rank=T, max_context_length=args.seq_len,
                                steps=steps_total, gc_freq=10 ** 6),
        parallelism=ParallelismConfig(data_parallel_shard_degree=-1, **par_overrides),
        checkpoint=CheckpointManager.Config(enable=False),
        activation_checkpoint=ActivationCheckpointConfig(mode=args.ac),
        kernels=KernelConfig(gemm=args.gemm, attention=args.attention),
    )
    cfg.debug.seed = 0
    cfg.debug.enable_structured_logging = False
    force_balance = bool(PRESETS[args.preset].get("force_balance", False))
    cfg.debug.moe_force_load_balance = force_balance
    if args.converters:
        cfg.model.converters = [c for c in args.converters.split(",") if c]
    trainer = cfg.build()
    for part in trainer.model_parts:
        # one sequence per microbatch is one document: no document mask is needed; with several sequences per
        # microbatch the positions restart and attention is masked per document
        part.single_document = args.local_batch == 1
    pd = trainer.pdims
    tokens_per_step = trainer.tokens_per_step_per_dp_rank * pd.dp_degree    # global tokens per optimizer step
    tokens_per_rank_step = trainer.tokens_per_step_per_dp_rank              # host -> device per step on a data rank
    layout = f"pp{pd.pp} dp_replicate{pd.dp_replicate} dp_shard{pd.dp_shard} cp{pd.cp} tp{pd.tp} ep{pd.ep}"
    dev = trainer.device
    mem = trainer.engines[0].memory_summary()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    it = trainer.batch_generator(trainer.dataloader)
    trainer.metrics_processor.should_log = lambda step: False  # logging syncs are measured explicitly below

    # ------------------------------------------------------------ end-to-end
    e2e = None
    h2d = d2h = 0
    if not args.skip_e2e:
        for _ in range(args.warmup):
            trainer.step += 1
            trainer.train_step(it)
            float(trainer._last_loss)
        barrier()
        t0 = time.perf_counter()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            trainer.step += 1
            trainer.train_step(it)  # pulls a pinned batch, copies it to the device, full optimizer step
            loss_host = float(trainer._last_loss)  # device -> host read of the step's result
        ev1.record()
        barrier()
        wall = time.perf_counter() - t0
        e2e_s = max_over_ranks(max(wall, ev0.elapsed_time(ev1) / 1e3))
        h2d = 3 * tokens_per_rank_step * 8  # input ids, positions, labels: int64 each
        d2h = 4
        e2e = {"value": tokens_per_step * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s / args.steps, "last_loss": loss_host}

    # ------------------------------------------------------------ device-timed
    class _Resident:
        """Feeds device-resident batches (inputs never leave the GPU): a different batch every step, so the loss
        stays that of unseen random tokens instead of a memorised batch."""

        def __init__(self, batches):
            self.batches = [({k: v.to(dev) for k, v in inp.items()}, lab.to(dev)) for inp, lab in batches]
            self.i = 0

        def __iter__(self):
            return self

        def __next__(self):
            b = self.batches[self.i % len(self.batches)]
            self.i += 1
            return b

    per_step = trainer.gradient_accumulation_steps * (cfg.parallelism.num_pp_microbatches if pd.pp_enabled else 1)
    resident = _Resident([next(it) for _ in range(min(64, (args.warmup + args.steps) * per_step))])
    for _ in range(args.warmup):
        trainer.step += 1
        trainer.train_step(resident)
    sampler = ClockSampler(dev.index or 0)
    OF.settings.launches = 0
    OF.settings.count_launches = True
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        trainer.step += 1
        trainer.train_step(resident)
    ev1.record()
    barrier()
    clocks = sampler.stop()
    OF.settings.count_launches = False
    launches = OF.settings.launches
    dev_s = max_over_ranks(ev0.elapsed_time(ev1) / 1e3)
    tokens_per_s = tokens_per_step * args.steps / dev_s
    peak = torch.cuda.max_memory_allocated(dev) / (1 << 30)
    flops_per_token = trainer.metrics_processor.num_flops_per_token
    loss_t = trainer._last_loss.detach().float().reshape(1).clone()
    lg = trainer.pdims.group("loss")
    if lg is not None:
        dist.all_reduce(loss_t, group=lg)   # every rank holds its share of the global mean
    if pd.pp_enabled:
        dist.all_reduce(loss_t, group=pd.group("pp"))   # only the last pipeline stage holds the loss
    loss = float(loss_t)
    if rank == 0:
        line = {
            "metric": "tokens_per_sec", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dev_s / args.steps,
            "higher_is_better": True, "scaling": "weak",
            # the published number is the bf16 FSDP headline; other presets have no published counterpart
            "vs_baseline": (tokens_per_s / world / BASELINE_TOKENS_PER_SEC_PER_GPU
                            if args.preset == "fsdp" and not args.converters and args.flavor == "8B" else None),
            "dtype": "bf16" if not args.converters else f"{args.converters} linears, bf16 elsewhere",
            "data": "synthetic uniform-random tokens (a new batch every step), random-init weights",
            "impl": "native",
            "tokens_per_sec_per_gpu": tokens_per_s / world,
            "mfu_pct": 100.0 * flops_per_token * tokens_per_s / world / 2.25e15,
            "tflops_per_gpu": flops_per_token * tokens_per_s / world / 1e12,
            "config": {"model": f"{args.model}-{args.flavor}", "global_batch": tokens_per_step // args.seq_len,
                       "seq_len": args.seq_len, "parallelism": f"fsdp{world}" if args.preset == "fsdp" else layout,
                       "preset": args.preset, "comm": args.comm, "tokens_per_step": tokens_per_step,
                       "activation_checkpoint": args.ac,
                       "optimizer": f"AdamW fp32 master, {args.opt_state} moments", "fsdp_comm": trainer.engines[0].comm if trainer.engines[0]._symm is None else "nvlink",
                       "gemm": args.gemm, "attention": args.attention,
                       "doc_mask": ("skipped (the microbatch is one sequence = one document)" if args.local_batch == 1 else
                                    f"on ({args.local_batch} sequences per microbatch, attention masked per document)"),
                       **({"moe_routing": "round-robin expert assignment (debug.moe_force_load_balance): balanced load on "
                                          "every step, the router's scores still weight the outputs"} if force_balance else {}),
                       "ac_policy": "selective = GEMM and attention outputs kept, norm outputs and SwiGLU activations "
                                    "recomputed in backward (no GEMM is recomputed)",
                       "param_layout": trainer.engines[0].param_layout(),
                       "l2": "per-step working set >> 126 MB L2 (no flush needed)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "peak_mem_gib": peak, "engine_mem_gib": mem, "loss": loss,
        }
        print(json.dumps(line), flush=True)
    trainer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
