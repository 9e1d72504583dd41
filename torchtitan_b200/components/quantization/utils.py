"""Shared pieces of the quantisation converters (parity: torchtitan/components/quantization/utils.py)."""

from __future__ import annotations

import dataclasses

__all__ = ["swap_linears", "iter_linear_configs", "module_filter"]

_SKIP = ("lm_head", "router", "gate", "tok_embeddings")


def iter_linear_configs(cfg, prefix="model"):
    """Yield ``(fqn, owner, attribute_or_index, linear_config)`` for every Linear config in the tree."""
    from torchtitan_b200.models.common.layers import Linear

    seen = set()

    def walk(node, path):
        if id(node) in seen or not dataclasses.is_dataclass(node):
            return
        seen.add(id(node))
        for f in dataclasses.fields(node):
            val = getattr(node, f.name, None)
            if isinstance(val, Linear.Config):
                yield path + "." + f.name, node, f.name, val
            elif dataclasses.is_dataclass(val):
                yield from walk(val, path + "." + f.name)
            elif isinstance(val, (list, tuple)):
                for i, item in enumerate(val):
                    if dataclasses.is_dataclass(item):
                        yield from walk(item, f"{path}.{f.name}.{i}")

    yield from walk(cfg, prefix)


def module_filter(fqn: str, lin, include) -> bool:
    """Linears that may be quantised: listed (or all), not the head / router, dimensions % 32 == 0
    once known (the owner fills the sizes in at build time, unknown sizes pass)."""
    if any(s in fqn for s in _SKIP):
        return False
    if include is not None and not any(s in fqn for s in include):
        return False
    return not ((lin.in_features and lin.in_features % 32) or (lin.out_features and lin.out_features % 32))


def swap_linears(model_cfg, *, recipe: str, include=None, **extra) -> int:
    from .linear import QuantLinear

    n = 0
    for fqn, owner, attr, lin in list(iter_linear_configs(model_cfg)):
        if type(lin).__qualname__ != "Linear.Config" or not module_filter(fqn, lin, include):
            continue
        kw = {f.name: getattr(lin, f.name) for f in dataclasses.fields(lin)}
        setattr(owner, attr, QuantLinear.Config(recipe=recipe, **extra, **kw))
        n += 1
    if n == 0:
        raise ValueError("the quantisation converter matched no Linear layer")
    return n


def mxfp8_converter(model_cfg, arg, job_config) -> int:
    """MXFP8: swaps the selected ``Linear`` configs for block-scaled fp8 linears (parity:
    torchtitan/components/quantization/mx.py:50-98).  ``arg``: comma-separated FQN substrings to include (default: every
    attention / MLP linear)."""
    fqns = [a for a in (arg or "").split(",") if a and a != "emulate"]
    return swap_linears(model_cfg, recipe="mxfp8", include=fqns or None)


def float8_converter(model_cfg, arg, job_config) -> int:
    """Float8 row-wise (parity: torchtitan/components/quantization/float8.py:53-173).  ``float8`` scales all three
    GEMMs row-wise, ``float8:rowwise_with_gw_hp`` keeps the weight-gradient GEMM in bf16; ``emulate`` is accepted for
    interface parity (the fp8 numerics are always reproduced exactly, see ``quantization.linear``)."""
    opts = [a for a in (arg or "").split(",") if a]
    hp = "rowwise_with_gw_hp" in opts
    fqns = [a for a in opts if a not in ("emulate", "rowwise", "rowwise_with_gw_hp")]
    return swap_linears(model_cfg, recipe="float8_rowwise", include=fqns or None, high_precision_wgrad=hp)
