"""Mergeable metric records for the RL loops.

Rollout workers, the batcher and the trainer loop each emit ``Metric(key, value)`` records; a value carries the
partial sums needed to merge it with other records of the same key and kind (so a mean over several sources is
the mean of all observations, not a mean of means).  ``aggregate`` groups records by ``(key, kind)``, merges each
group and returns the flat ``{"key/suffix": float}`` dict that goes to the console, a JSONL file and the
framework's metric loggers.

Kinds: ``Mean`` (``/mean``), ``Max`` (``/max``), ``Min`` (``/min``), ``Sum`` (``/sum``), ``Std`` (population,
``/std``), ``SummaryStats`` (``/_max /_mean /_min /_std /_sum``: underscore names never collide with the single
kinds under the same key) and ``NoReduce`` (an already reduced value: exactly one record per key, emitted under
the bare key).  Empty observations reduce to NaN (sum: 0).

Parity: torchtitan/experiments/rl/observability/metrics/types.py:30-386 (value kinds),
processor.py:36-226 (aggregation + backends), console.py:38-136 (allow-list and formatting),
controller_metrics.py:20-54 (step timer).
"""

from __future__ import annotations

import fnmatch
import json
import math
import os
import time
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, ClassVar, Iterable, Sequence

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

__all__ = ["Metric", "MetricValue", "Mean", "Max", "Min", "Sum", "Std", "SummaryStats", "NoReduce", "aggregate",
           "MetricsTimer", "MetricsProcessor", "format_metric_value"]

_NAN = float("nan")


class MetricValue:
    """Moments of a set of observations: count, sum, sum of squares, min, max.  Every kind keeps all five (a few
    floats) and differs only in what ``emit`` reports after the merge."""

    suffix: ClassVar[str] = ""
    __slots__ = ("count", "total", "sumsq", "lo", "hi")

    def __init__(self, value: float, count: float = 1.0):
        v = float(value)
        self.count, self.total = float(count), v
        self.sumsq = v * v if count == 1 else _NAN      # unknown for a pre-aggregated sum unless given by the subclass
        self.lo = self.hi = v if count == 1 else _NAN

    @classmethod
    def from_list(cls, values: Iterable[Any]) -> "MetricValue":
        xs = [float(v) for v in values]
        out = cls.__new__(cls)
        out.count, out.total = float(len(xs)), sum(xs)
        out.sumsq = sum(x * x for x in xs)
        out.lo, out.hi = (min(xs), max(xs)) if xs else (_NAN, _NAN)
        return out

    def merge(self, other: "MetricValue") -> None:
        self.count += other.count
        self.total += other.total
        self.sumsq += other.sumsq
        # NaN-aware: an empty record must not poison the extrema of the others
        self.lo = other.lo if math.isnan(self.lo) else (self.lo if math.isnan(other.lo) else min(self.lo, other.lo))
        self.hi = other.hi if math.isnan(self.hi) else (self.hi if math.isnan(other.hi) else max(self.hi, other.hi))

    @classmethod
    def reduce(cls, records: Sequence["MetricValue"]) -> dict[str, float]:
        acc = cls.from_list([])
        for r in records:
            acc.merge(r)
        return acc.emit()

    # -- what each kind reports ------------------------------------------------------------------------------------
    def _mean(self) -> float:
        return self.total / self.count if self.count else _NAN

    def _std(self) -> float:
        if not self.count:
            return _NAN
        mu = self.total / self.count
        return math.sqrt(max(0.0, self.sumsq / self.count - mu * mu))

    def emit(self) -> dict[str, float]:
        raise NotImplementedError

    def __repr__(self) -> str:
        return f"{type(self).__name__}(count={self.count:g}, total={self.total:g})"


class Mean(MetricValue):
    """``Mean(x)`` one observation, ``Mean(total, count=n)`` pre-aggregated, ``Mean.from_list(xs)``."""
    suffix = "mean"

    def emit(self):
        return {self.suffix: self._mean()}


class Max(MetricValue):
    suffix = "max"

    def emit(self):
        return {self.suffix: self.hi}


class Min(MetricValue):
    suffix = "min"

    def emit(self):
        return {self.suffix: self.lo}


class Sum(MetricValue):
    suffix = "sum"

    def emit(self):
        return {self.suffix: self.total}


class Std(MetricValue):
    """Population standard deviation.  ``Std(total, count=n, sum_squares=s)`` takes pre-aggregated moments: both or
    neither of ``count`` / ``sum_squares``."""
    suffix = "std"

    def __init__(self, value: float, *, count: float | None = None, sum_squares: float | None = None):
        if (count is None) != (sum_squares is None):
            raise ValueError("Std needs both count and sum_squares for pre-aggregated input")
        super().__init__(value, 1.0 if count is None else count)
        if sum_squares is not None:
            self.sumsq = float(sum_squares)

    def emit(self):
        return {self.suffix: self._std()}


class SummaryStats(MetricValue):
    def emit(self):
        if not self.count:
            return {"_max": _NAN, "_mean": _NAN, "_min": _NAN, "_std": _NAN, "_sum": 0.0}
        return {"_max": self.hi, "_mean": self._mean(), "_min": self.lo, "_std": self._std(), "_sum": self.total}


class NoReduce(MetricValue):
    """A value that is already final (a loss the trainer reduced over its ranks, a gauge): one record per key."""

    @classmethod
    def from_list(cls, values):
        xs = list(values)
        if len(xs) > 1:
            raise ValueError(f"NoReduce holds exactly one value, got {len(xs)}")
        return super().from_list(xs)

    @classmethod
    def reduce(cls, records):
        if len(records) != 1:
            raise ValueError(f"NoReduce expects exactly one record per key, got {len(records)}")
        return {"": records[0].total}

    def emit(self):
        return {"": self.total}


@dataclass
class Metric:
    """``Metric("rollout/response_length", Max.from_list([12, 18, 9]))``: the emitted name is ``key/suffix``, so the
    same key may carry several kinds."""
    key: str
    value: MetricValue


def aggregate(metrics: Iterable[Metric]) -> dict[str, float]:
    groups: dict[tuple[str, type], list[MetricValue]] = {}
    for m in metrics:
        groups.setdefault((m.key, type(m.value)), []).append(m.value)
    out: dict[str, float] = {}
    for (key, kind), records in groups.items():
        try:
            reduced = kind.reduce(records)
        except ValueError as e:
            raise ValueError(f"metric '{key}': {e}") from None
        for suffix, v in reduced.items():
            out[key if suffix == "" else f"{key}/{suffix}"] = v
    return out


class MetricsTimer:
    """``with timer.record("timing/step/optim"): ...`` accumulates wall time per key; ``flush`` returns the records
    and starts over."""

    def __init__(self):
        self._t: dict[str, float] = {}

    @contextmanager
    def record(self, key: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self._t[key] = self._t.get(key, 0.0) + time.perf_counter() - t0

    def flush(self) -> list[Metric]:
        out = [Metric(k, NoReduce(v)) for k, v in self._t.items()]
        self._t = {}
        return out


def format_metric_value(v: float) -> str:
    if isinstance(v, float) and math.isnan(v):
        return "nan"
    a = abs(v)
    if a != 0 and (a >= 1e5 or a < 1e-3):
        return f"{v:.3e}"
    return f"{v:.4g}" if float(v) != int(v) else str(int(v))


class MetricsProcessor(Configurable):
    """Aggregates a step's records and hands the flat dict to the console (filtered by an allow-list of glob
    patterns), to ``<dump_folder>/rl_metrics.jsonl`` and to any extra logger with a ``log(metrics, step)`` method
    (the framework's TensorBoard / W&B container fits).  Validation records are prefixed ``validation/``."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        console_allow: list[str] = field(default_factory=lambda: ["loss*", "reward*", "rollout_reward*", "timing/step/total",
                                                                   "policy_age*", "advantage/_mean", "optim/*"])
        """Glob patterns of the metric names printed per step (everything is written to the file)."""
        jsonl: bool = True

    def __init__(self, config: Config | None = None, *, dump_folder: str | None = None, loggers: Sequence[Any] = ()):
        self.config = config or MetricsProcessor.Config()
        self.loggers = list(loggers)
        self.history: list[dict] = []
        self._path = None
        if dump_folder and self.config.jsonl:
            os.makedirs(dump_folder, exist_ok=True)
            self._path = os.path.join(dump_folder, "rl_metrics.jsonl")

    def log(self, *, step: int, metrics: Iterable[Metric], is_validation: bool = False) -> dict[str, float]:
        flat = aggregate(metrics)
        if is_validation:
            flat = {(k if k.startswith("validation/") else f"validation/{k}"): v for k, v in flat.items()}
        self.history.append({"step": step, **flat})
        shown = {k: v for k, v in sorted(flat.items())
                 if any(fnmatch.fnmatch(k, pat) or fnmatch.fnmatch(k, "validation/" + pat) for pat in self.config.console_allow)}
        if shown:
            logger.info(f"{'val ' if is_validation else ''}step {step}: "
                        + "  ".join(f"{k}={format_metric_value(v)}" for k, v in shown.items()))
        if self._path:
            with open(self._path, "a") as f:
                f.write(json.dumps({"step": step, "validation": is_validation,
                                    **{k: (None if isinstance(v, float) and math.isnan(v) else v) for k, v in flat.items()}}) + "\n")
        for lg in self.loggers:
            lg.log(flat, step)
        return flat
