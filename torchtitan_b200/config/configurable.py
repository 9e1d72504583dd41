"""Component/config pairing used by every buildable part of the framework.

A component class derives from :class:`Configurable` and declares a nested
``Config`` dataclass.  ``Config.build(**runtime)`` constructs the owning
component, ``Config.walk`` enumerates nested configs of a given type together
with a handle that lets the caller swap them (this is what model converters and
the override mechanism use), and ``Config.to_dict`` produces a JSON-safe dump.

Behavioural parity: torchtitan/config/configurable.py:18-180 (the reference
enforces ``kw_only``/``slots`` dataclasses, auto-wires ``build`` to the owner
class and rejects runtime kwargs that shadow config fields).
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, fields, is_dataclass
from typing import Any, Callable, ClassVar, Iterator

__all__ = ["Configurable", "ConfigRef", "config_to_dict", "Function"]


def config_to_dict(value: Any) -> Any:
    """Recursively convert configs / dataclasses / containers to JSON-safe data."""
    if isinstance(value, Configurable.Config):
        return value.to_dict()
    if is_dataclass(value) and not isinstance(value, type):
        return {
            f.name: config_to_dict(getattr(value, f.name))
            for f in fields(value)
            if not f.name.startswith("_")
        }
    if isinstance(value, (list, tuple)):
        return [config_to_dict(v) for v in value]
    if isinstance(value, dict):
        return {str(k): config_to_dict(v) for k, v in value.items()}
    if isinstance(value, (str, int, float, bool)) or value is None:
        return value
    return repr(value)


@dataclass
class ConfigRef:
    """Location of a nested config: ``holder[key]`` (attribute or list index)."""

    fqn: str
    config: Any
    holder: Any  # dataclass instance, list or dict that stores the config (None for the root)
    key: Any  # attribute name / list index / dict key

    def replace(self, new_config: Any) -> None:
        if self.holder is None:
            raise ValueError("the root config cannot be replaced through a ConfigRef")
        if isinstance(self.holder, (list, dict)):
            self.holder[self.key] = new_config
        else:
            setattr(self.holder, self.key, new_config)
        self.config = new_config


class Configurable:
    """Base class of all components that are constructed from a ``Config``."""

    @dataclass(kw_only=True, slots=True)
    class Config:
        _owner: ClassVar[type | None] = None

        # -- construction -------------------------------------------------
        def build(self, **runtime: Any):
            owner = type(self)._owner
            if owner is None:
                raise TypeError(f"{type(self).__qualname__} is not attached to a component class")
            names = {f.name for f in fields(self)}
            clash = names.intersection(runtime)
            if clash:
                raise TypeError(
                    f"runtime arguments {sorted(clash)} shadow fields of {type(self).__qualname__}"
                )
            return owner(self, **runtime)

        # -- introspection ------------------------------------------------
        def to_dict(self) -> dict:
            return {
                f.name: config_to_dict(getattr(self, f.name))
                for f in fields(self)
                if not f.name.startswith("_")
            }

        def walk(self, config_cls: type | tuple[type, ...], *, descend_into_matches: bool = False,
                 prefix: str = "") -> Iterator[ConfigRef]:
            """Yield a :class:`ConfigRef` for every nested config of ``config_cls``.

            The FQN of a ref equals the module FQN that ``build`` would create
            (``layers.3.feed_forward.w1``).  Lists and dicts are traversed.
            """
            yield from _walk(self, config_cls, descend_into_matches, prefix, None, None)

        # kept for users coming from the reference API
        def traverse(self, config_cls, *, recurse: bool = False, _prefix: str = ""):
            for ref in self.walk(config_cls, descend_into_matches=recurse, prefix=_prefix):
                yield ref.fqn, ref.config, ref.holder, ref.key

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        cfg = cls.__dict__.get("Config")
        if cfg is None or cfg.__qualname__ != f"{cls.__qualname__}.Config":
            return      # no own Config, or an alias of another component's Config (which keeps its owner)
        if not is_dataclass(cfg):
            raise TypeError(f"{cls.__qualname__}.Config must be a dataclass")
        params = getattr(cfg, "__dataclass_params__", None)
        if params is not None and not getattr(params, "kw_only", True):
            raise TypeError(f"{cls.__qualname__}.Config must be declared with kw_only=True")
        cfg._owner = cls

    def __init__(self, config: "Configurable.Config", **_: Any):
        self.config = config


def _walk(node, config_cls, descend, prefix, holder, key) -> Iterator[ConfigRef]:
    if isinstance(node, config_cls):
        yield ConfigRef(prefix, node, holder, key)
        if not descend:
            return
    if is_dataclass(node) and not isinstance(node, type):
        for f in fields(node):
            if f.name.startswith("_"):
                continue
            child = getattr(node, f.name)
            child_fqn = f"{prefix}.{f.name}" if prefix else f.name
            yield from _walk_value(child, config_cls, descend, child_fqn, node, f.name)


def _walk_value(value, config_cls, descend, fqn, holder, key) -> Iterator[ConfigRef]:
    if is_dataclass(value) and not isinstance(value, type):
        yield from _walk(value, config_cls, descend, fqn, holder, key)
    elif isinstance(value, list):
        for i, item in enumerate(value):
            yield from _walk_value(item, config_cls, descend, f"{fqn}.{i}", value, i)
    elif isinstance(value, dict):
        for k, item in value.items():
            yield from _walk_value(item, config_cls, descend, f"{fqn}.{k}", value, k)


def replace_config(cfg, **changes):
    """``dataclasses.replace`` that tolerates slots dataclasses and ClassVars."""
    return dataclasses.replace(cfg, **changes)


Factory = Callable[..., Any]


class Function(Configurable):
    """Any callable as a config node: ``Function.Config(fn=...).build()`` is itself callable.  For config fields
    whose value is computed when the owner is built, e.g. a per-layer initialiser that depends on the depth
    (parity: torchtitan/config/function.py:16-40)."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        fn: Callable[..., Any]

    def __init__(self, config: "Function.Config", **_: Any):
        self.fn = config.fn

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self.fn(*args, **kwargs)
