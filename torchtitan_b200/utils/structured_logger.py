"""Per-rank structured trace: spans, instants and scalars as JSON lines.

Every record carries ``rank``, ``source``, ``time_us``, ``step``, ``relative_step``
(steps since the process started) and the tags attached to the current step
(``gc``, ``eval``, ``checkpoint_save``).  Records go to
``<output_dir>/structured_logs/rank<r>.jsonl``; extra sinks can be plugged with
:func:`add_handler`.  :func:`to_chrome_trace` merges rank files into one
chrome://tracing document (Gantt view).  Parity:
torchtitan/observability/structured_logger/*.py.
"""

from __future__ import annotations

import contextlib
import glob
import json
import os
import threading
import time
from typing import Any, Callable

__all__ = ["init_structured_logger", "span", "log_trace_span", "log_trace_instant", "log_trace_scalar",
           "set_step", "add_step_tag", "add_handler", "close", "to_chrome_trace", "enabled"]

_lock = threading.Lock()
_handlers: list[Callable[[dict], None]] = []
_file = None
_state = {"rank": 0, "source": "", "step": 0, "first_step": None, "tags": [], "enabled": False}


def enabled() -> bool:
    return _state["enabled"]


def init_structured_logger(source: str, output_dir: str, rank: int | None = None, enable: bool = True) -> None:
    global _file
    close()
    _state.update(rank=int(os.environ.get("RANK", "0")) if rank is None else rank, source=source,
                  step=0, first_step=None, tags=[], enabled=enable)
    if not enable:
        return
    d = os.path.join(output_dir, "structured_logs")
    os.makedirs(d, exist_ok=True)
    _file = open(os.path.join(d, f"rank{_state['rank']}.jsonl"), "a", buffering=1 << 16)
    factories = os.environ.get("TITAN_STRUCT_LOGGER_HANDLERS", "")
    for spec in filter(None, (s.strip() for s in factories.split(","))):
        import importlib

        mod, _, fn = spec.rpartition(".")
        _handlers.append(getattr(importlib.import_module(mod), fn)())


def add_handler(fn: Callable[[dict], None]) -> None:
    _handlers.append(fn)
    _state["enabled"] = True


def close() -> None:
    global _file
    with _lock:
        if _file is not None:
            _file.flush()
            _file.close()
            _file = None
        _handlers.clear()
        _state["enabled"] = False


def set_step(step: int) -> None:
    _state["step"] = step
    if _state["first_step"] is None:
        _state["first_step"] = step
    _state["tags"] = []


def add_step_tag(tag: str) -> None:
    if tag not in _state["tags"]:
        _state["tags"].append(tag)


def _emit(kind: str, name: str, **extra: Any) -> None:
    if not _state["enabled"]:
        return
    first = _state["first_step"]
    rec = {"kind": kind, "name": name, "rank": _state["rank"], "source": _state["source"],
           "time_us": time.time_ns() // 1000, "step": _state["step"],
           "relative_step": (_state["step"] - first) if first is not None else 0,
           "step_tags": list(_state["tags"])}
    rec.update(extra)
    with _lock:
        if _file is not None:
            _file.write(json.dumps(rec) + "\n")
        for h in _handlers:
            h(rec)


@contextlib.contextmanager
def span(name: str, **attrs: Any):
    if not _state["enabled"]:
        yield
        return
    _emit("span_start", name, **attrs)
    t0 = time.perf_counter_ns()
    try:
        yield
    finally:
        _emit("span_end", name, dur_us=(time.perf_counter_ns() - t0) // 1000, **attrs)


log_trace_span = span


def log_trace_instant(name: str, **attrs: Any) -> None:
    _emit("instant", name, **attrs)


def log_trace_scalar(name: str, value: float, **attrs: Any) -> None:
    _emit("scalar", name, value=value, **attrs)


def to_chrome_trace(log_dir: str, out_path: str) -> int:
    """Merge ``rank*.jsonl`` under ``log_dir`` into a chrome trace; returns the event count."""
    events = []
    for path in sorted(glob.glob(os.path.join(log_dir, "rank*.jsonl"))):
        open_spans: dict[str, list[dict]] = {}
        with open(path) as f:
            for line in f:
                r = json.loads(line)
                base = {"pid": r["rank"], "tid": r["source"], "name": r["name"],
                        "args": {"step": r["step"], "tags": r["step_tags"]}}
                if r["kind"] == "span_start":
                    open_spans.setdefault(r["name"], []).append(r)
                elif r["kind"] == "span_end":
                    stack = open_spans.get(r["name"])
                    if stack:
                        s = stack.pop()
                        events.append(dict(base, ph="X", ts=s["time_us"], dur=r.get("dur_us", r["time_us"] - s["time_us"])))
                elif r["kind"] == "instant":
                    events.append(dict(base, ph="i", ts=r["time_us"], s="p"))
                elif r["kind"] == "scalar":
                    events.append({"pid": r["rank"], "name": r["name"], "ph": "C", "ts": r["time_us"],
                                   "args": {r["name"]: r["value"]}})
    with open(out_path, "w") as f:
        json.dump({"traceEvents": events}, f)
    return len(events)
