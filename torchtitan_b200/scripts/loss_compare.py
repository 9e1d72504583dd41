"""Compare the loss curves of two training configurations, step by step.

    python -m torchtitan_b200.scripts.loss_compare --steps 10 \
        --baseline "--module llama3 --config llama3_debugmodel" \
        --test     "--module llama3 --config llama3_debugmodel --parallelism.tensor_parallel_degree 2" \
        [--assert-equal] [--tolerance 1e-6] [--export golden.json | --import golden.json]

Both runs use deterministic mode, the same seed and synthetic or file data with the same order.
With more than one process (``torchrun``) every rank takes part and rank 0 reports.  ``--export``
stores the baseline losses, ``--import`` compares the test run against stored losses instead of
running the baseline.  Parity: scripts/loss_compare.py:1-120.
"""

from __future__ import annotations

import argparse
import json
import shlex
import sys
import tempfile


def run_losses(arg_string: str, steps: int, seed: int) -> list[float]:
    from torchtitan_b200.config import ConfigManager

    with tempfile.TemporaryDirectory() as tmp:
        argv = shlex.split(arg_string) + [
            "--training.steps", str(steps), "--debug.seed", str(seed), "--debug.deterministic",
            "--debug.no-enable_structured_logging", "--checkpoint.no-enable", "--dump_folder", tmp]
        trainer = ConfigManager().parse_args(argv).build()
        losses = []
        it = trainer.batch_generator(trainer.dataloader)
        try:
            for _ in range(steps):
                trainer.step += 1
                trainer.train_step(it)
                losses.append(float(trainer._last_loss))
        finally:
            trainer.close()
    return losses


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--baseline", default="")
    ap.add_argument("--test", required=True)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--assert-equal", action="store_true")
    ap.add_argument("--tolerance", type=float, default=0.0)
    ap.add_argument("--export", dest="export_path")
    ap.add_argument("--import", dest="import_path")
    args = ap.parse_args(argv)
    if args.import_path:
        with open(args.import_path) as f:
            base = json.load(f)["losses"]
    else:
        if not args.baseline:
            ap.error("--baseline or --import is required")
        base = run_losses(args.baseline, args.steps, args.seed)
    if args.export_path:
        with open(args.export_path, "w") as f:
            json.dump({"args": args.baseline, "seed": args.seed, "losses": base}, f, indent=2)
    test = run_losses(args.test, args.steps, args.seed)
    worst = 0.0
    print(f"{'step':>5} {'baseline':>14} {'test':>14} {'diff':>12}")
    for i, (a, b) in enumerate(zip(base, test), 1):
        worst = max(worst, abs(a - b))
        print(f"{i:5d} {a:14.8f} {b:14.8f} {b - a:12.3e}")
    print(f"max |diff| = {worst:.3e}")
    if args.assert_equal and worst > args.tolerance:
        print("FAILED: the loss curves differ", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
