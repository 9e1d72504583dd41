"""Config-tree overrides: swap component configs selected by type and FQN glob.

An override is a function decorated with :func:`override`.  It receives the
config found at a matching location and returns the replacement.  Overrides are
named on the command line (``--override.imports pkg.mod.fn`` or
``pkg.mod.fn={"rank": 4}``), collected first and applied afterwards so that two
overrides touching the same node, or a node and one of its ancestors, are
reported as a conflict instead of silently depending on order.

Parity: torchtitan/config/override.py:60-515.
"""

from __future__ import annotations

import fnmatch
import importlib
import json
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Callable

from .configurable import ConfigRef

__all__ = ["OverrideConfig", "override", "derive", "apply_overrides", "OverrideConflict", "registered_overrides"]


class OverrideConflict(RuntimeError):
    pass


@dataclass(kw_only=True, slots=True)
class OverrideConfig:
    imports: list[str] = field(default_factory=list)
    """Entries ``module.function`` or ``module.function={json kwargs}``."""


@dataclass
class _Spec:
    name: str
    fn: Callable[..., Any]
    target: type
    fqns: tuple[str, ...]
    exact: bool


_REGISTRY: dict[str, _Spec] = {}


def override(*, target: type, fqns: list[str] | tuple[str, ...] = ("*",), exact: bool = False):
    """Register ``fn(cfg, **kwargs) -> new_cfg`` for configs of type ``target``.

    ``fqns`` are globs over the config FQN; with ``exact=True`` only configs whose
    type is exactly ``target`` (not subclasses) are replaced.
    """

    def deco(fn):
        name = f"{fn.__module__}.{fn.__qualname__}"
        _REGISTRY[name] = _Spec(name, fn, target, tuple(fqns), exact)
        fn.__override_name__ = name
        return fn

    return deco


def registered_overrides() -> dict[str, _Spec]:
    return dict(_REGISTRY)


def derive(src: Any, target_cls: type, **deltas: Any):
    """Build ``target_cls`` copying every field it shares with ``src``."""
    shared = {}
    tnames = {f.name for f in fields(target_cls) if f.init}
    for f in fields(src):
        if f.name in tnames and f.name not in deltas:
            shared[f.name] = getattr(src, f.name)
    shared.update(deltas)
    return target_cls(**shared)


def _parse_import(entry: str) -> tuple[str, dict]:
    name, eq, payload = entry.partition("=")
    kwargs = json.loads(payload) if eq else {}
    if not isinstance(kwargs, dict):
        raise ValueError(f"override arguments must be a JSON object: {entry}")
    return name.strip(), kwargs


def _resolve(name: str) -> _Spec:
    if name not in _REGISTRY:
        mod_name, _, _fn = name.rpartition(".")
        if not mod_name:
            raise ValueError(f"override '{name}' must be a dotted path")
        importlib.import_module(mod_name)
    if name not in _REGISTRY:
        raise ValueError(f"'{name}' is not a registered @override function")
    return _REGISTRY[name]


def apply_overrides(root: Any, imports: list[str]) -> list[tuple[str, str]]:
    """Apply the named overrides to every matching node below ``root``.

    Returns ``[(fqn, override_name)]`` of replaced nodes.
    """
    planned: dict[str, tuple[ConfigRef, _Spec, dict]] = {}
    for entry in imports:
        name, kwargs = _parse_import(entry)
        spec = _resolve(name)
        matched = False
        for ref in root.walk(spec.target, descend_into_matches=True):
            if ref.holder is None:
                continue
            if spec.exact and type(ref.config) is not spec.target:
                continue
            if not any(fnmatch.fnmatchcase(ref.fqn, g) for g in spec.fqns):
                continue
            matched = True
            if ref.fqn in planned and planned[ref.fqn][1].name != spec.name:
                raise OverrideConflict(
                    f"'{ref.fqn}' is claimed by both {planned[ref.fqn][1].name} and {spec.name}"
                )
            planned[ref.fqn] = (ref, spec, kwargs)
        if not matched:
            raise ValueError(f"override {name} matched no config node")
    fqns = sorted(planned)
    for a in fqns:
        for b in fqns:
            if a != b and b.startswith(a + "."):
                raise OverrideConflict(
                    f"'{a}' ({planned[a][1].name}) is an ancestor of '{b}' ({planned[b][1].name})"
                )
    done = []
    for fqn in fqns:
        ref, spec, kwargs = planned[fqn]
        new_cfg = spec.fn(ref.config, **kwargs)
        if new_cfg is None or not is_dataclass(new_cfg):
            raise TypeError(f"override {spec.name} must return a config dataclass")
        ref.replace(new_cfg)
        done.append((fqn, spec.name))
    return done
