"""Model converters: config-tree rewrites applied before the model is built.

``apply_converters(model_cfg, names, job_config)`` runs them in order; quantization
converters must precede ``lora`` (parity: torchtitan/models/utils.py:23-42).
"""

from __future__ import annotations

__all__ = ["apply_converters", "CONVERTERS", "has_quantization"]

QUANT = ("mxfp8", "float8", "nvfp4", "mxfp8_experts", "float8_experts")


def _lm_head_cast(cfg, arg, job):
    # imported on use: the converter lives with the RL experiment, which the core must not load otherwise
    from torchtitan_b200.experiments.rl.cast_linear import lm_head_cast_converter

    return lm_head_cast_converter(cfg, arg, job)


def _registry():
    from .utils import float8_converter, mxfp8_converter
    from torchtitan_b200.components.lora import lora_converter

    from .grouped import quantize_experts
    from .nvfp4 import nvfp4_converter

    return {"lm_head_cast": _lm_head_cast, "mxfp8": mxfp8_converter, "float8": float8_converter, "lora": lora_converter,
            "nvfp4": nvfp4_converter,
            "mxfp8_experts": lambda cfg, arg, job: quantize_experts(cfg, "mxfp8"),
            "float8_experts": lambda cfg, arg, job: quantize_experts(cfg, "float8_rowwise")}


CONVERTERS = ("mxfp8", "float8", "nvfp4", "mxfp8_experts", "float8_experts", "lora", "lm_head_cast")


def has_quantization(names) -> bool:
    return any(n.split(":")[0] in QUANT for n in names)


def apply_converters(model_cfg, names, job_config=None) -> None:
    if not names:
        return
    reg = _registry()
    seen_lora = False
    for entry in names:
        name, _, arg = entry.partition(":")
        if name not in reg:
            raise ValueError(f"unknown model converter '{name}' (have {sorted(reg)})")
        if name == "lora":
            seen_lora = True
        elif seen_lora and name in QUANT:
            raise ValueError("quantization converters must come before 'lora'")
        reg[name](model_cfg, arg, job_config)
