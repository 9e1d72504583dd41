"""Entry point of RL jobs::

    python -m torchtitan_b200.experiments.rl.train --module rl --config rl_grpo_debug_alphabet_sort \\
        [--controller.async_loop.num_training_steps 20 --trainer.optimizer.lr 3e-4 ...]
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m torchtitan_b200.experiments.rl.train --module rl --config ...

Parity: torchtitan/experiments/rl/train.py:421-476 (main).
"""

from __future__ import annotations

import sys

from torchtitan_b200.config import ConfigManager
from torchtitan_b200.utils.logging import init_logger, logger


def main(argv: list[str] | None = None):
    init_logger()
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--module" not in argv and not any(a.startswith("--module=") for a in argv):
        argv = ["--module", "rl", "--config", "rl_grpo_debug_alphabet_sort", *argv]
    cfg = ConfigManager().parse_args(argv)
    job = cfg.build()
    try:
        out = job.run()
        if out is not None:
            for k in sorted(k for k in out["post"] if "reward" in k and k.endswith("_mean")):
                logger.info(f"{k}: {out['pre'].get(k, float('nan')):.4f} -> {out['post'][k]:.4f}")
        return out
    finally:
        job.close()


if __name__ == "__main__":
    main()
