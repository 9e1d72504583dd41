"""MXFP8 converter: swaps the selected ``Linear`` configs of a model config tree for block-scaled
fp8 linears (parity: torchtitan/components/quantization/mx.py:50-98; the grouped-expert variant of
:104-206 maps to ``GroupedExperts`` running on fake-quantised rows)."""

from __future__ import annotations

from .utils import swap_linears


def mxfp8_converter(model_cfg, arg, job_config) -> int:
    """``arg``: comma-separated FQN substrings to include (default: every attention / MLP linear)."""
    fqns = [a for a in (arg or "").split(",") if a and a != "emulate"]
    return swap_linears(model_cfg, recipe="mxfp8", include=fqns or None)
