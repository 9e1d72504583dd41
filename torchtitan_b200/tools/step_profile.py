"""Device-time breakdown of one training step by kernel.

    python -m torchtitan_b200.tools.step_profile --module llama3 --config llama3_8b [--top 30] [overrides ...]

Builds the trainer from a registered config on synthetic data, runs three warm-up steps, records
the CUDA activity of the next step with the PyTorch profiler (device timeline only) and prints
the kernels sorted by total device time with their launch counts and shares.  Trailing arguments
are ordinary config overrides (``--model.converters mxfp8``, ``--training.max_context_length 4096``).
"""

from __future__ import annotations

import argparse
import os


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--module", default="llama3")
    ap.add_argument("--config", default="llama3_8b")
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    args, extra = ap.parse_known_args(argv)
    os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
    import torch
    from torch.profiler import ProfilerActivity, profile

    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.utils.logging import init_logger

    init_logger()
    cfg = ConfigManager().parse_args([
        "--module", args.module, "--config", args.config, "--dataloader.dataset", "synthetic", "--training.steps", "100",
        "--metrics.log_freq", "1000000", "--debug.seed", "0", "--debug.no-enable_structured_logging",
        "--checkpoint.no-enable", "--dump_folder", "/tmp/tb200_step_profile"] + extra)
    trainer = cfg.build()
    tr = cfg.training
    # one sequence per microbatch is one document; several sequences keep their per-document attention mask
    trainer.model.single_document = tr.num_tokens_per_microbatch_per_dp_rank <= tr.max_context_length
    it = trainer.batch_generator(trainer.dataloader)
    for _ in range(args.warmup):
        trainer.step += 1
        trainer.train_step(it)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.step += 1
        trainer.train_step(it)
        torch.cuda.synchronize()
    rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
    total = sum(e.device_time_total for e in rows)
    if int(os.environ.get("RANK", "0")) != 0:     # under torchrun every rank profiles its own step; rank 0 reports
        trainer.close()
        return 0
    print(f"total device time {total / 1e3:.1f} ms over {sum(e.count for e in rows)} launches")
    for e in rows[: args.top]:
        print(f"{e.device_time_total / 1e3:9.2f} ms {100 * e.device_time_total / total:5.1f}% n={e.count:5d}  {e.key[:110]}")
    trainer.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
