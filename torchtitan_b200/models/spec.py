"""Model registry protocol.

A model family package exposes ``model_registry(flavor) -> ModelSpec``.  The spec
bundles the architecture config with the functions that parallelise it, split it
into pipeline stages and translate its checkpoints to Hugging Face names.
Parity: torchtitan/protocols/model_spec.py:32-76, torchtitan/models/__init__.py:7-18.
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any, Callable

__all__ = ["ModelSpec", "get_model_spec", "SUPPORTED_MODELS"]

SUPPORTED_MODELS = ("llama3", "qwen3", "deepseek_v3", "gpt_oss", "kimi_k2_7", "muse_glimmer", "qwen3_5", "flux")


@dataclass
class ModelSpec:
    name: str
    flavor: str
    model: Any  # Decoder.Config (or another root Module.Config)
    parallelize_fn: Callable | None = None
    pipelining_fn: Callable | None = None
    post_optimizer_build_fn: Callable | None = None
    state_dict_adapter: type | None = None

    def walk(self, config_cls, **kw):
        yield from self.model.walk(config_cls, prefix="model", **kw)


def _truncate_layers(spec: ModelSpec, n: int) -> ModelSpec:
    cfg = spec.model
    layers = getattr(cfg, "layers", None)
    if not isinstance(layers, list) or not 0 < n <= len(layers):
        raise ValueError(f"cannot keep {n} layers of {spec.name} {spec.flavor}")
    cfg.layers = layers[-n:] if n < len(layers) else layers   # the last layers: the mixture-of-experts ones of mixed stacks
    for i, blk in enumerate(cfg.layers):
        if hasattr(blk, "layer_id"):
            blk.layer_id = i
    if hasattr(cfg, "n_layers"):
        cfg.n_layers = n
    spec.flavor = f"{spec.flavor}@{n}"
    return spec


def get_model_spec(name: str, flavor: str) -> ModelSpec:
    """``flavor`` may end in ``@N``: the architecture with only N of its layers (per-layer cost of a large model on
    a few GPUs: profiling and benchmarks; not a registered training recipe)."""
    if "@" in flavor:
        base, n = flavor.rsplit("@", 1)
        return _truncate_layers(get_model_spec(name, base), int(n))
    for root in ("torchtitan_b200.models", "torchtitan_b200.experiments"):
        try:
            mod = importlib.import_module(f"{root}.{name}")
        except ModuleNotFoundError:
            continue
        return mod.model_registry(flavor)
    raise ValueError(f"unknown model '{name}' (supported: {SUPPORTED_MODELS})")
