"""Command line → config tree.

Three sources are merged, later ones winning:

1. a registry function ``--module llama3 --config llama3_8b`` returning a
   ``Trainer.Config`` (parity: torchtitan/config/manager.py:34-159);
2. a TOML job file ``--job.config_file path.toml`` whose tables are the config
   sections (``[training]``, ``[parallelism]``, ``[model]`` ...);
3. dotted overrides ``--training.steps 20 --checkpoint.enable
   --metrics.no-enable_tensorboard``.

Strings are converted using the dataclass field annotations, so the same code
handles TOML values and CLI strings.  ``list[str]`` fields accept a
comma-separated value.
"""

from __future__ import annotations

import dataclasses
import importlib
import json
import sys
import tomllib
import types
import typing
from dataclasses import fields, is_dataclass
from typing import Any, Callable, get_args, get_origin, get_type_hints

__all__ = ["ConfigManager", "apply_dotted_overrides", "apply_mapping", "ConfigError"]


class ConfigError(ValueError):
    pass


_TRUE = {"1", "true", "yes", "on"}
_FALSE = {"0", "false", "no", "off"}


def _strip_annotated(tp):
    while get_origin(tp) is typing.Annotated:
        tp = get_args(tp)[0]
    return tp


def _coerce(value: Any, tp: Any, where: str) -> Any:
    """Convert ``value`` (TOML object or CLI string) to annotation ``tp``."""
    tp = _strip_annotated(tp)
    origin = get_origin(tp)
    if tp is Any or tp is object:
        return value
    if origin in (typing.Union, types.UnionType):
        options = [a for a in get_args(tp)]
        if value is None or (isinstance(value, str) and value.lower() in ("none", "null")):
            if type(None) in options:
                return None
        last_err: Exception | None = None
        for opt in options:
            if opt is type(None):
                continue
            try:
                return _coerce(value, opt, where)
            except (ConfigError, ValueError, TypeError) as e:  # try next alternative
                last_err = e
        raise ConfigError(f"{where}: cannot interpret {value!r} as {tp}: {last_err}")
    if origin is typing.Literal:
        choices = get_args(tp)
        for c in choices:
            if value == c or (isinstance(value, str) and str(c) == value):
                return c
        raise ConfigError(f"{where}: {value!r} is not one of {choices}")
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str):
            if value.lower() in _TRUE:
                return True
            if value.lower() in _FALSE:
                return False
        raise ConfigError(f"{where}: expected a boolean, got {value!r}")
    if tp is int:
        if isinstance(value, bool):
            raise ConfigError(f"{where}: expected int, got bool")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            return int(value.replace("_", ""), 0)
        raise ConfigError(f"{where}: expected int, got {value!r}")
    if tp is float:
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        if isinstance(value, str):
            return float(value)
        raise ConfigError(f"{where}: expected float, got {value!r}")
    if tp is str:
        if isinstance(value, str):
            return value
        raise ConfigError(f"{where}: expected str, got {value!r}")
    if origin in (list, tuple) or tp in (list, tuple):
        args = get_args(tp)
        elem = args[0] if args else Any
        if isinstance(value, str):
            text = value.strip()
            if text.startswith("["):
                value = json.loads(text)
            else:
                value = [v for v in (s.strip() for s in text.split(",")) if v != ""]
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{where}: expected a list, got {value!r}")
        out = [_coerce(v, elem, f"{where}[{i}]") for i, v in enumerate(value)]
        return tuple(out) if (origin is tuple or tp is tuple) else out
    if origin is dict or tp is dict:
        if isinstance(value, str):
            value = json.loads(value)
        if not isinstance(value, dict):
            raise ConfigError(f"{where}: expected a table, got {value!r}")
        return dict(value)
    if is_dataclass(tp):
        if isinstance(value, tp):
            return value
        if isinstance(value, dict):
            inst = tp()
            apply_mapping(inst, value, where)
            return inst
        raise ConfigError(f"{where}: expected a table for {tp.__name__}")
    return value


def _hints(obj) -> dict[str, Any]:
    cls = type(obj)
    try:
        return get_type_hints(cls, include_extras=True)
    except Exception:
        return {f.name: f.type for f in fields(cls)}


def apply_mapping(cfg: Any, table: dict, where: str = "") -> None:
    """Merge a (possibly nested) mapping, e.g. a parsed TOML table, into ``cfg``."""
    hints = _hints(cfg)
    names = {f.name for f in fields(cfg)}
    for key, value in table.items():
        loc = f"{where}.{key}" if where else key
        if key not in names:
            raise ConfigError(f"unknown config key '{loc}' (known: {sorted(names)})")
        current = getattr(cfg, key)
        if isinstance(value, dict) and is_dataclass(current):
            apply_mapping(current, value, loc)
        else:
            setattr(cfg, key, _coerce(value, hints.get(key, Any), loc))


def _set_dotted(cfg: Any, dotted: str, value: Any) -> None:
    parts = dotted.split(".")
    node = cfg
    for i, p in enumerate(parts[:-1]):
        if isinstance(node, list):
            node = node[int(p)]
        elif isinstance(node, dict):
            node = node[p]
        elif is_dataclass(node) and hasattr(node, p):
            node = getattr(node, p)
        else:
            raise ConfigError(f"unknown config path '{'.'.join(parts[: i + 1])}'")
    leaf = parts[-1]
    negate = False
    if is_dataclass(node) and not hasattr(node, leaf):
        for pre in ("no-", "no_"):
            if leaf.startswith(pre) and hasattr(node, leaf[len(pre):]):
                leaf, negate = leaf[len(pre):], True
                break
    if isinstance(node, list):
        node[int(leaf)] = value
        return
    if isinstance(node, dict):
        node[leaf] = value
        return
    if not (is_dataclass(node) and hasattr(node, leaf)):
        raise ConfigError(f"unknown config option '--{dotted}'")
    hint = _hints(node).get(leaf, Any)
    if negate:
        if value is not None:
            raise ConfigError(f"'--{dotted}' takes no value")
        setattr(node, leaf, False)
        return
    if value is None:
        base = _strip_annotated(hint)
        if base is bool or (get_origin(base) in (typing.Union, types.UnionType) and bool in get_args(base)):
            setattr(node, leaf, True)
            return
        raise ConfigError(f"'--{dotted}' needs a value")
    setattr(node, leaf, _coerce(value, hint, dotted))


def apply_dotted_overrides(cfg: Any, argv: list[str]) -> None:
    """Apply ``--a.b value``, ``--a.b=value``, ``--a.flag`` and ``--a.no-flag``."""
    i = 0
    while i < len(argv):
        tok = argv[i]
        if not tok.startswith("--"):
            raise ConfigError(f"unexpected argument {tok!r}")
        body = tok[2:]
        value: Any = None
        if "=" in body:
            body, value = body.split("=", 1)
        elif i + 1 < len(argv) and not _looks_like_flag(argv[i + 1]):
            value = argv[i + 1]
            i += 1
        _set_dotted(cfg, body, value)
        i += 1


def _looks_like_flag(tok: str) -> bool:
    if not tok.startswith("--"):
        return False
    return len(tok) > 2 and not tok[2].isdigit()


_MODULE_ROOTS = ("torchtitan_b200.models", "torchtitan_b200.experiments")


class ConfigManager:
    """Builds the root ``Trainer.Config`` from argv."""

    def __init__(self, default_factory: Callable[[], Any] | None = None):
        self._default_factory = default_factory
        self.config: Any = None

    # -- registry lookup ---------------------------------------------------
    @staticmethod
    def load_registry_fn(module: str, config: str) -> Callable[[], Any]:
        candidates = [f"{root}.{module}.config_registry" for root in _MODULE_ROOTS]
        candidates += [f"{module}.config_registry", module]
        errors = []
        for name in candidates:
            try:
                mod = importlib.import_module(name)
            except ModuleNotFoundError as e:
                errors.append(f"{name}: {e}")
                continue
            fn = getattr(mod, config, None)
            if callable(fn):
                return fn
            errors.append(f"{name}: no function '{config}'")
        raise ConfigError("cannot resolve --module %s --config %s:\n  %s" % (module, config, "\n  ".join(errors)))

    def parse_args(self, argv: list[str] | None = None):
        argv = list(sys.argv[1:] if argv is None else argv)
        module = config_fn = toml_path = None
        rest: list[str] = []
        i = 0
        while i < len(argv):
            tok = argv[i]
            key, eq, val = tok.partition("=")
            if key in ("--module", "--config", "--job.config_file", "--job.config-file", "--config_file"):
                if not eq:
                    if i + 1 >= len(argv):
                        raise ConfigError(f"{key} needs a value")
                    val = argv[i + 1]
                    i += 1
                if key == "--module":
                    module = val
                elif key == "--config":
                    config_fn = val
                else:
                    toml_path = val
            else:
                rest.append(tok)
            i += 1

        if module is not None or config_fn is not None:
            if module is None or config_fn is None:
                raise ConfigError("--module and --config must be given together")
            cfg = self.load_registry_fn(module, config_fn)()
        else:
            if self._default_factory is None:
                from torchtitan_b200.trainer import Trainer

                cfg = Trainer.Config()
            else:
                cfg = self._default_factory()

        if toml_path is not None:
            with open(toml_path, "rb") as f:
                table = tomllib.load(f)
            table.pop("job", None) if "job" in table and not hasattr(cfg, "job") else None
            apply_mapping(cfg, table)
        apply_dotted_overrides(cfg, rest)
        validate = getattr(cfg, "validate", None)
        if callable(validate):
            validate()
        self.config = cfg
        return cfg


def main(argv: list[str] | None = None) -> None:
    """``python -m torchtitan_b200.config.manager [args]`` prints the resolved config."""
    cfg = ConfigManager().parse_args(argv)
    print(json.dumps(cfg.to_dict(), indent=2, default=str))


if __name__ == "__main__":
    main()
