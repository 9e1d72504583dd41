"""Kineto traces and CUDA memory snapshots.

``Profiler`` is a context manager around the train loop; ``step()`` is called after
every optimizer step.  Traces go to
``<dump_folder>/<save_traces_folder>/iteration_<step>/rank<r>_trace.json.gz``;
memory snapshots (python stacks) are pickled every ``memory_snapshot_freq`` steps and
on ``torch.OutOfMemoryError``.  Parity: torchtitan/tools/profiler.py:24-395.
"""

from __future__ import annotations

import contextlib
import os
import pickle
import time
from dataclasses import dataclass
from typing import Any

import torch

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

__all__ = ["Profiler"]


class Profiler(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        enable_profiling: bool = False
        save_traces_folder: str = "profiling/traces"
        profile_freq: int = 10
        profiler_repeat: int | None = None
        profiler_skip_first: int | None = None
        profiler_skip_first_wait: int | None = None
        profiler_active: int = 1
        profiler_warmup: int = 3
        enable_memory_snapshot: bool = False
        memory_snapshot_freq: int | None = None
        save_memory_snapshot_folder: str = "profiling/memory_snapshot"
        memory_snapshot_max_entries: int = 1_000_000
        trace_post_processor: Any = None

    def __init__(self, config: "Profiler.Config", *, global_step: int = 0, base_folder: str = "./outputs",
                 rank: int = 0, **_):
        self.config = config
        self.rank = rank
        self.base = base_folder
        self.step_num = global_step
        self._prof = None
        self._mem = False

    def __enter__(self):
        c = self.config
        if c.enable_profiling:
            warmup, active = c.profiler_warmup, c.profiler_active
            wait = c.profile_freq - (active + warmup)
            if wait < 0:
                raise ValueError("profile_freq must be >= profiler_warmup + profiler_active")
            trace_dir = os.path.join(self.base, c.save_traces_folder)
            os.makedirs(trace_dir, exist_ok=True)

            def on_ready(prof):
                d = os.path.join(trace_dir, f"iteration_{self.step_num}")
                os.makedirs(d, exist_ok=True)
                path = os.path.join(d, f"rank{self.rank}_trace.json.gz")
                t = time.monotonic()
                prof.export_chrome_trace(path)
                logger.info(f"Dumped profiler trace {path} in {time.monotonic() - t:.2f}s")
                if c.trace_post_processor is not None:
                    fn = c.trace_post_processor.build() if hasattr(c.trace_post_processor, "build") else c.trace_post_processor
                    fn(path)

            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            kw = {}
            if c.profiler_skip_first is not None:
                kw["skip_first"] = c.profiler_skip_first
            if c.profiler_skip_first_wait is not None:
                kw["skip_first_wait"] = c.profiler_skip_first_wait
            self._prof = torch.profiler.profile(
                activities=acts,
                schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active,
                                                 repeat=c.profiler_repeat or 0, **kw),
                on_trace_ready=on_ready, record_shapes=True)
            self._prof.__enter__()
            self._prof.step_num = self.step_num
        if c.enable_memory_snapshot and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=c.memory_snapshot_max_entries, stacks="python")
            self._mem = True
        return self

    def _dump_memory(self, suffix: str = "") -> None:
        d = os.path.join(self.base, self.config.save_memory_snapshot_folder, f"iteration_{self.step_num}{suffix}")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, f"rank{self.rank}_memory_snapshot.pickle"), "wb") as f:
            pickle.dump(torch.cuda.memory._snapshot(), f)
        logger.info(f"Dumped memory snapshot to {d}")

    def step(self) -> None:
        self.step_num += 1
        if self._prof is not None:
            self._prof.step()
        freq = self.config.memory_snapshot_freq
        if self._mem and freq and self.step_num % freq == 0:
            self._dump_memory()

    def __exit__(self, exc_type, exc, tb):
        if self._mem and exc_type is not None and issubclass(exc_type, torch.OutOfMemoryError):
            self._dump_memory("_exit")
        if self._prof is not None:
            self._prof.__exit__(exc_type, exc, tb)
        if self._mem:
            torch.cuda.memory._record_memory_history(enabled=None)
        return False
