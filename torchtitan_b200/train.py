"""Entry point: ``python -m torchtitan_b200.train --module llama3 --config llama3_8b [--a.b v]``
or ``python -m torchtitan_b200.train --job.config_file job.toml``.

Flow (parity: torchtitan/train.py:17-79): logger -> config -> structured logger ->
build trainer -> (seed checkpoint | train) -> close, destroy the process group.
"""

from __future__ import annotations

import os
import sys

import torch

from torchtitan_b200.config import ConfigManager
from torchtitan_b200.utils import structured_logger as sl
from torchtitan_b200.utils.logging import init_logger, logger


def main(argv: list[str] | None = None) -> None:
    init_logger()
    from torchtitan_b200.trainer import Trainer
    from torchtitan_b200.parallel import utils as dist_utils

    config = ConfigManager().parse_args(argv)
    debug = getattr(config, "debug", None)
    sl.init_structured_logger("training", getattr(config, "dump_folder", "./outputs"),
                              enable=bool(debug and debug.enable_structured_logging))
    if getattr(getattr(config, "comm", None), "mode", "default") == "local_tensor":
        # one process emulates every rank and checks the sharding plan; nothing is trained (as in the reference)
        from torchtitan_b200.parallel.local_plan import validate_plan

        validate_plan(config)
        return
    trainer = None
    seed_ckpt = bool(getattr(getattr(config, "checkpoint", None), "create_seed_checkpoint", False))
    try:
        if seed_ckpt:
            if int(os.environ.get("WORLD_SIZE", "1")) != 1:
                raise RuntimeError("a seed checkpoint must be created by a single process")
            if not config.checkpoint.enable:
                raise RuntimeError("checkpoint.create_seed_checkpoint needs checkpoint.enable")
        trainer = config.build()   # the LLM trainer, or a family's own trainer (e.g. flux)
        if seed_ckpt:
            trainer.checkpointer.create_seed_checkpoint()
        else:
            trainer.train()
    except Exception:
        logger.exception("training failed")
        raise
    finally:
        if trainer is not None:
            trainer.close()
        sl.close()
        dist_utils.destroy()


if __name__ == "__main__":
    main()
