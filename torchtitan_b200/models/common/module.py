"""Module protocol shared by all model parts.

* ``Module`` = ``nn.Module`` + :class:`Configurable`: every layer is built from a
  nested ``Config`` so config-tree rewrites (quantization, LoRA, overrides) can
  retarget it before construction.
* Parameters carry an :class:`InitSpec`.  Initial values are a pure function of
  ``(seed, parameter FQN)``; they do not depend on how the parameter is sharded,
  which is what makes 1-rank vs N-rank runs and seed checkpoints agree.  (The
  reference gets the same property from DTensor's RNG, torchtitan/trainer.py:489-494,
  torchtitan/protocols/module.py:72-119.)
* ``checkpoint_slices`` lets a module expose row-slices of a fused parameter
  under the un-fused checkpoint names (``wqkv`` -> ``wq``/``wk``/``wv``).
"""

from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from typing import Iterator

import torch
import torch.nn as nn

from torchtitan_b200.config import Configurable

__all__ = ["Module", "InitSpec", "set_init", "materialize_param", "ModuleDict", "ModuleList", "fqn_seed"]


@dataclass(frozen=True)
class InitSpec:
    kind: str = "normal"  # normal | trunc_normal | ones | zeros | uniform | constant
    mean: float = 0.0
    std: float = 0.02
    a: float = -2.0
    b: float = 2.0
    value: float = 0.0


def set_init(param: torch.Tensor, spec: InitSpec) -> None:
    param._init_spec = spec  # type: ignore[attr-defined]


def fqn_seed(seed: int, fqn: str) -> int:
    h = hashlib.sha256(f"{seed}:{fqn}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def materialize_param(shape, spec: InitSpec, seed: int, fqn: str, device="cpu") -> torch.Tensor:
    """Full fp32 initial value of a parameter (always generated on CPU for portability
    of the random stream, then moved)."""
    shape = tuple(shape)
    if spec.kind == "ones":
        return torch.ones(shape, dtype=torch.float32, device=device)
    if spec.kind == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    if spec.kind == "constant":
        return torch.full(shape, spec.value, dtype=torch.float32, device=device)
    # The stream is generated on the target device type (Philox on CUDA, MT on CPU): values
    # are reproducible per device type and independent of the parallel layout.
    gdev = torch.device(device) if torch.device(device).type == "cuda" else torch.device("cpu")
    gen = torch.Generator(device=gdev)
    gen.manual_seed(fqn_seed(seed, fqn))
    t = torch.empty(shape, dtype=torch.float32, device=gdev)
    if spec.kind == "normal":
        t.normal_(spec.mean, spec.std, generator=gen)
    elif spec.kind == "trunc_normal":
        nn.init.trunc_normal_(t, mean=spec.mean, std=spec.std, a=spec.a, b=spec.b, generator=gen)
    elif spec.kind == "uniform":
        t.uniform_(spec.a, spec.b, generator=gen)
    else:
        raise ValueError(f"unknown init kind {spec.kind}")
    return t.to(device)


class Module(nn.Module, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    def __init__(self, config=None, **_):
        nn.Module.__init__(self)
        self.config = config

    # ---- initialisation ------------------------------------------------
    def init_states(self, seed: int = 0, prefix: str = "") -> None:
        """Initialise all parameters in place (single-process path).

        The sharded engine does not call this for parameters; it materialises
        each full parameter and scatters it into its fp32 shards.
        """
        with torch.no_grad():
            for name, p in self.named_parameters():
                spec = getattr(p, "_init_spec", None) or InitSpec()
                fqn = f"{prefix}{name}"
                p.copy_(materialize_param(p.shape, spec, seed, fqn).to(p.dtype))
        self.init_buffers()

    def init_buffers(self, device=None) -> None:
        """Recreate non-persistent buffers (RoPE tables); recursive."""
        for m in self.children():
            if isinstance(m, Module):
                m.init_buffers(device)
            else:
                for sub in m.children() if isinstance(m, (nn.ModuleDict, nn.ModuleList)) else []:
                    if isinstance(sub, Module):
                        sub.init_buffers(device)

    # ---- checkpoint naming ----------------------------------------------
    def checkpoint_slices(self) -> dict[str, list[tuple[str, int, int]]]:
        """``{local_param_name: [(checkpoint_name, row_start, row_end), ...]}`` for fused params."""
        return {}


class ModuleDict(nn.ModuleDict):
    pass


class ModuleList(nn.ModuleList):
    pass


def iter_checkpoint_slices(model: nn.Module) -> Iterator[tuple[str, list[tuple[str, int, int]]]]:
    """Yield ``(param_fqn, [(ckpt_fqn, r0, r1)])`` for every fused parameter of ``model``."""
    for mod_name, mod in model.named_modules():
        fn = getattr(mod, "checkpoint_slices", None)
        if fn is None:
            continue
        for local, pieces in fn().items():
            pre = f"{mod_name}." if mod_name else ""
            yield pre + local, [(pre + n, a, b) for n, a, b in pieces]
