"""Float8 row-wise converter (parity: torchtitan/components/quantization/float8.py:53-173).
``float8`` = row-wise scaling for all three GEMMs, ``float8:rowwise_with_gw_hp`` keeps the weight
gradient GEMM in bf16; ``emulate`` is accepted for interface parity (the fp8 numerics are always
reproduced exactly, see ``quantization.linear``)."""

from __future__ import annotations

from .utils import swap_linears


def float8_converter(model_cfg, arg, job_config) -> int:
    opts = [a for a in (arg or "").split(",") if a]
    hp = "rowwise_with_gw_hp" in opts
    fqns = [a for a in opts if a not in ("emulate", "rowwise", "rowwise_with_gw_hp")]
    return swap_linears(model_cfg, recipe="float8_rowwise", include=fqns or None, high_precision_wgrad=hp)
