"""Console logging: ``[titan] time - logger - level - message`` (parity: torchtitan/tools/logging.py)."""

from __future__ import annotations

import logging
import os

logger = logging.getLogger("torchtitan_b200")
_warned: set[str] = set()


def init_logger(level: int | None = None) -> logging.Logger:
    if level is None:
        level = getattr(logging, os.environ.get("TITAN_LOG_LEVEL", "INFO").upper(), logging.INFO)
    logger.setLevel(level)
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("[titan] %(asctime)s - %(name)s - %(levelname)s - %(message)s"))
        logger.addHandler(h)
        logger.propagate = False
    return logger


def warn_once(msg: str) -> None:
    if msg not in _warned:
        _warned.add(msg)
        logger.warning(msg)


class Color:
    black = "\033[30m"; red = "\033[31m"; green = "\033[32m"; yellow = "\033[33m"; blue = "\033[34m"
    magenta = "\033[35m"; cyan = "\033[36m"; white = "\033[37m"; reset = "\033[39m"; orange = "\033[38;2;180;60;0m"
    turquoise = "\033[38;2;54;234;195m"


class NoColor:
    black = red = green = yellow = blue = magenta = cyan = white = reset = orange = turquoise = ""
