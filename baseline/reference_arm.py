"""Reference arm of the benchmark: the unmodified upstream torchtitan, driven through its own
``Trainer`` (``torchtitan/train.py``), on the same metric and config as the native arm.

Nothing from ``torchtitan_b200`` is imported here.  Two installs are tried, in this order:

1. ``baseline/_ref`` -- the reference source tree (0.2.2) installed offline with pip.  Its trainer
   imports ``spmd_types``, ``grain``, ``torchao`` and PyTorch-nightly FSDP symbols; when any of
   them is missing the import error is kept as ``ref_0_2_2_unavailable``.
2. the torchtitan that ships in the image's site-packages (0.1.0, same project, unmodified).

Either is run on its stock path: Llama-3 8B from its own registry, FSDP2 (``fully_shard``, bf16
parameters / fp32 reduce) over all ranks, per-op selective activation checkpointing, per-block
``torch.compile``, fused AdamW, gradient clipping at 1.0.  Upstream reads its C4 sample and its
tokenizer from files that do not exist offline, so the arm registers a second ``TrainSpec`` (the
upstream extension point, ``torchtitan/protocols/train_spec.py``) that differs from the stock
``llama3`` one only in the data loader and the tokenizer: uniform-random token ids of the same
shape from pinned host memory, exactly what the native arm trains on.

Timing follows the native arm: W warm-up steps, then K steps between CUDA events with a barrier
and a synchronize on both sides, max over ranks; ``value`` with the batch resident on the device
and logging off, ``e2e`` with a fresh pinned batch copied to the device each step and upstream's
own per-step metric logging on (``metrics.log_freq = 1``: it reads loss and grad-norm back to the
host every step).
"""

from __future__ import annotations

import dataclasses
import json
import os
import socket
import sys
import time

BASELINE_TOKENS_PER_SEC_PER_GPU = 8307.5


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _purge_torchtitan_modules() -> None:
    for k in [k for k in sys.modules if k == "torchtitan" or k.startswith("torchtitan.")]:
        del sys.modules[k]


def _import_reference(root: str) -> dict:
    """Returns {"version", "source", "note"} after making ``import torchtitan`` resolve to a usable install."""
    ref_dir = os.path.join(root, "baseline", "_ref")
    note = None
    if os.path.isdir(os.path.join(ref_dir, "torchtitan")):
        sys.path.insert(0, ref_dir)
        try:
            import torchtitan.trainer  # noqa: F401  (0.2.2's public training API)

            return {"version": "0.2.2", "source": "baseline/_ref", "note": None, "api": "0.2"}
        except Exception as e:
            note = f"baseline/_ref (0.2.2) not importable: {type(e).__name__}: {str(e)[:160]}"
            sys.path.remove(ref_dir)
            _purge_torchtitan_modules()
    else:
        note = "baseline/_ref is empty"
    import importlib.metadata as md

    import torchtitan.train  # noqa: F401  (the image-installed release)

    return {"version": md.version("torchtitan"), "source": os.path.dirname(sys.modules["torchtitan"].__file__),
            "note": note, "api": "0.1"}


def _register_synthetic_spec(vocab_size: int):
    """A TrainSpec equal to upstream's ``llama3`` except for the data loader and the tokenizer."""
    import torch
    from torchtitan.components.dataloader import BaseDataLoader
    from torchtitan.components.tokenizer import BaseTokenizer
    from torchtitan.protocols.train_spec import get_train_spec, register_train_spec

    class SyntheticLoader(BaseDataLoader):
        """Uniform-random token ids; every batch is a new pinned host tensor."""

        def __init__(self, batch: int, seq: int, seed: int):
            self.batch, self.seq = batch, seq
            self.gen = torch.Generator().manual_seed(seed)

        def __iter__(self):
            while True:
                ids = torch.randint(0, vocab_size, (self.batch, self.seq + 1), generator=self.gen, dtype=torch.int64)
                inp = ids[:, :-1].contiguous().pin_memory()
                lab = ids[:, 1:].contiguous().pin_memory()
                yield {"input": inp}, lab

        def state_dict(self):
            return {}

        def load_state_dict(self, sd):
            pass

    class StubTokenizer(BaseTokenizer):
        def encode(self, *a, **k):
            return []

        def decode(self, *a, **k):
            return ""

        def get_vocab_size(self):
            return vocab_size

    def build_loader(dp_world_size, dp_rank, tokenizer, job_config, **_):
        return SyntheticLoader(job_config.training.local_batch_size, job_config.training.seq_len, seed=1234 + dp_rank)

    base = get_train_spec("llama3")
    spec = dataclasses.replace(base, name="llama3_synthetic", build_dataloader_fn=build_loader,
                               build_tokenizer_fn=lambda job_config: StubTokenizer(), build_validator_fn=None)
    register_train_spec(spec)
    return spec


class _Resident:
    """Feeds one device-resident batch every step."""

    def __init__(self, batch, device):
        inp, lab = batch
        self.inp = {k: v.to(device) for k, v in inp.items()}
        self.lab = lab.to(device)

    def __iter__(self):
        return self

    def __next__(self):
        return dict(self.inp), self.lab


def run(args, root: str, clock_sampler_cls) -> None:
    rank = int(os.environ.setdefault("RANK", "0"))
    os.environ.setdefault("LOCAL_RANK", "0")
    world = int(os.environ.setdefault("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        os.environ["MASTER_PORT"] = str(_free_port())
    os.environ.setdefault("TORCHINDUCTOR_CACHE_DIR", "/tmp/tb200_ref_inductor")
    out = {"impl": "reference"}

    def fail(msg: str) -> None:
        if rank == 0:
            out["unavailable"] = msg[:400]
            print(json.dumps(out), flush=True)

    if world != args.gpus:
        return fail(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    try:
        info = _import_reference(root)
    except Exception as e:
        return fail(f"no importable torchtitan install: {type(e).__name__}: {e}")
    if info["api"] != "0.1":
        return fail("baseline/_ref imported, but this arm only drives the 0.1 Trainer API")

    import torch
    import torch.distributed as dist
    from torchtitan.config import ConfigManager
    from torchtitan.train import Trainer

    if not torch.cuda.is_available():
        return fail("no CUDA device")
    flavor = args.flavor
    compile_on = os.environ.get("TB200_REF_COMPILE", "1") != "0"
    steps_total = 10 ** 6
    cli = [
        "--model.name", "llama3_synthetic", "--model.flavor", flavor,
        "--job.dump_folder", "/tmp/tb200_ref_out",
        "--training.seq_len", str(args.seq_len), "--training.local_batch_size", str(args.local_batch),
        "--training.steps", str(steps_total), "--training.max_norm", "1.0", "--training.seed", "0",
        "--training.mixed_precision_param", "bfloat16", "--training.mixed_precision_reduce", "float32",
        "--training.gc_freq", str(10 ** 6),
        "--parallelism.data_parallel_shard_degree", "-1",
        "--optimizer.name", "AdamW", "--optimizer.lr", "3e-4", "--optimizer.implementation", "fused",
        "--lr_scheduler.warmup_steps", "2",
        "--activation_checkpoint.mode", "selective" if args.ac == "selective" else args.ac,
        "--activation_checkpoint.selective_ac_option", "op",
        "--metrics.log_freq", str(10 ** 9),
    ]
    if compile_on:
        cli += ["--training.compile"]
    try:
        spec = _register_synthetic_spec(vocab_size=128256 if flavor != "debugmodel" else 2000)
        job_config = ConfigManager().parse_args(cli)
        trainer = Trainer(job_config)
    except Exception as e:
        return fail(f"reference Trainer could not be built: {type(e).__name__}: {e}")
    dev = trainer.device
    T = args.seq_len * args.local_batch

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

    step_error = None
    try:
        # ---------------------------------------------------------------- end to end
        it = trainer.batch_generator(trainer.dataloader)
        job_config.metrics.log_freq = 1  # upstream's logging reads loss and grad-norm back every step
        for _ in range(args.warmup):
            trainer.step += 1
            trainer.train_step(it)
        barrier()
        t0 = time.perf_counter()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            trainer.step += 1
            trainer.train_step(it)
        ev1.record()
        barrier()
        wall = time.perf_counter() - t0
        e2e_s = max_over_ranks(max(wall, ev0.elapsed_time(ev1) / 1e3))
        e2e = {"value": T * world * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * 8,
               "d2h_bytes_per_step": 8, "ms_per_step": 1e3 * e2e_s / args.steps}

        # ---------------------------------------------------------------- device-timed
        job_config.metrics.log_freq = 10 ** 9
        trainer.step = 10  # never 1 again: upstream always logs step 1
        resident = trainer.batch_generator(_Resident(next(iter(trainer.dataloader)), dev))
        for _ in range(max(1, args.warmup // 2)):
            trainer.step += 1
            trainer.train_step(resident)
        sampler = clock_sampler_cls(dev.index or 0)
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
        dev_s = max_over_ranks(ev0.elapsed_time(ev1) / 1e3)
    except Exception as e:  # an OOM or a compile failure inside the reference's own step
        step_error = f"{type(e).__name__}: {str(e)[:300]}"
    if step_error is not None:
        fail(f"reference train_step failed: {step_error}")
    else:
        tokens_per_s = T * world * args.steps / dev_s
        flops_per_token = trainer.metrics_processor.num_flops_per_token
        peak = torch.cuda.max_memory_allocated(dev) / (1 << 30)
        if rank == 0:
            out.update({
                "metric": "tokens_per_sec", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dev_s / args.steps,
                "higher_is_better": True, "scaling": "weak",
                "vs_baseline": tokens_per_s / world / BASELINE_TOKENS_PER_SEC_PER_GPU,
                "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
                "reference_version": f"{info['version']} ({info['source']})",
                "ref_0_2_2_unavailable": info["note"], "same_config": True,
                "tokens_per_sec_per_gpu": tokens_per_s / world,
                "mfu_pct": 100.0 * flops_per_token * tokens_per_s / world / 2.25e15,
                "config": {"model": f"llama3-{flavor}", "global_batch": args.local_batch * world, "seq_len": args.seq_len,
                           "parallelism": f"fsdp{world}" if world > 1 else "single GPU (upstream applies no FSDP at "
                           "dp_shard=1: fp32 parameters under bf16 autocast)",
                           "activation_checkpoint": "selective (per-op SAC)", "compile": compile_on,
                           "optimizer": "AdamW fused, fp32 states", "attention": "upstream SDPA",
                           "l2": "per-step working set >> 126 MB L2 (no flush needed)"},
                "clocks": clocks, "e2e": e2e, "peak_mem_gib": peak,
            })
            print(json.dumps(out), flush=True)
    try:
        trainer.close()
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception:
        pass
