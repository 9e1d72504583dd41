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


def get_model_spec(name: str, flavor: str) -> ModelSpec:
    for root in ("torchtitan_b200.models", "torchtitan_b200.experiments"):
        try:
            mod = importlib.import_module(f"{root}.{name}")
        except ModuleNotFoundError:
            continue
        return mod.model_registry(flavor)
    raise ValueError(f"unknown model '{name}' (supported: {SUPPORTED_MODELS})")
