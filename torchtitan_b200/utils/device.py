"""Device helpers: local device selection, peak-FLOPS table, capability probes, GC control.

Peak numbers are the dense bf16 tensor-core rates used for MFU (parity:
torchtitan/tools/utils.py:141-259; B200 = 2.25e15).
"""

from __future__ import annotations

import gc
import os
import time

import torch

from .logging import logger

__all__ = ["get_local_device", "get_peak_flops", "GarbageCollection", "has_cuda_capability", "device_name"]

_PEAK_BF16 = [
    ("GB300", 2.5e15), ("GB200", 2.5e15), ("B300", 2.25e15), ("B200", 2.25e15),
    ("H200", 989e12), ("H100 NVL", 835e12), ("H100 PCIe", 756e12), ("H100", 989e12),
    ("A100", 312e12), ("MI355X", 2.5e15), ("MI300X", 1.3e15), ("MI250X", 191.5e12), ("L40S", 362e12),
]


def get_local_device() -> torch.device:
    if torch.cuda.is_available():
        idx = int(os.environ.get("LOCAL_RANK", "0")) % max(1, torch.cuda.device_count())
        return torch.device("cuda", idx)
    return torch.device("cpu")


def device_name(device: torch.device | None = None) -> str:
    if device is not None and device.type == "cuda":
        return torch.cuda.get_device_name(device)
    return "cpu"


def get_peak_flops(name: str) -> float:
    for key, val in _PEAK_BF16:
        if key in name:
            return val
    if name != "cpu":
        logger.warning(f"peak FLOPS of '{name}' unknown, using the A100 figure for MFU")
    return 312e12


def has_cuda_capability(major: int, minor: int) -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (major, minor)


class GarbageCollection:
    """Disable automatic GC and collect generation 1 every ``gc_freq`` steps so that
    all ranks pause at the same step (parity: torchtitan/tools/utils.py:100-136)."""

    def __init__(self, gc_freq: int = 1000, debug: bool = False):
        assert gc_freq > 0, "gc_freq must be positive"
        self.gc_freq = gc_freq
        self.debug = debug
        gc.disable()
        self.collect("initial GC collection")
        if debug:
            from torch.utils.viz._cycles import warn_tensor_cycles

            warn_tensor_cycles()

    def run(self, step: int) -> bool:
        if self.debug:
            self.collect("GC collection invoked by debug mode", generation=2)
            gc.collect()
            return True
        if step > 1 and step % self.gc_freq == 0:
            self.collect("periodic GC collection")
            return True
        return False

    @staticmethod
    def collect(reason: str, generation: int = 1) -> None:
        t = time.monotonic()
        gc.collect(generation)
        logger.debug("[GC] %s took %.2f seconds", reason, time.monotonic() - t)
