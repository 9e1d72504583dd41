"""Output projection computed in a wider dtype than the parameters are stored and gathered in.

Token log-probabilities of the trainer are compared with those the generator recorded; the importance ratio is
sensitive to bf16 rounding of the logits, so RL configs run the ``lm_head`` matmul in fp32 on both sides:
``CastLinear`` casts input, weight and bias in ``forward`` (the stored parameter keeps its dtype, which keeps weight
tying and the sharded layout untouched) and ``lm_head_cast_converter`` swaps only the decoder's ``lm_head`` config,
so LoRA and the quantisation converters still see plain ``Linear`` everywhere else.  Registered as the model
converter ``lm_head_cast[:dtype]``.

Parity: torchtitan/experiments/rl/models/cast_linear.py:33-114.
"""

from __future__ import annotations

from dataclasses import dataclass, fields

import torch
import torch.nn.functional as F

from torchtitan_b200.models.common.layers import Linear

__all__ = ["CastLinear", "lm_head_cast_converter"]

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "float64": torch.float64}


class CastLinear(Linear):
    @dataclass(kw_only=True, slots=True)
    class Config(Linear.Config):
        compute_dtype: str = "float32"

    def __init__(self, config: "CastLinear.Config", **kw):
        super().__init__(config, **kw)
        if config.compute_dtype not in _DTYPES:
            raise ValueError(f"compute_dtype must be one of {sorted(_DTYPES)}, got {config.compute_dtype!r}")
        self.compute_dtype = _DTYPES[config.compute_dtype]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        d = self.compute_dtype
        return F.linear(x.to(d), self.weight.to(d), None if self.bias is None else self.bias.to(d))


def lm_head_cast_converter(model_cfg, arg: str = "", job_config=None) -> None:
    """Replace every ``Linear.Config`` named ``lm_head`` in the config tree by a ``CastLinear.Config`` with the
    same fields; ``arg`` is the compute dtype (default float32)."""
    found = 0
    for ref in list(model_cfg.walk(Linear.Config)):
        if ref.fqn.rsplit(".", 1)[-1] != "lm_head" or isinstance(ref.config, CastLinear.Config):
            continue
        shared = {f.name: getattr(ref.config, f.name) for f in fields(ref.config) if not f.name.startswith("_")}
        ref.replace(CastLinear.Config(**shared, compute_dtype=arg or "float32"))
        found += 1
    if not found:
        raise ValueError("lm_head_cast: the model config has no Linear named 'lm_head'")
