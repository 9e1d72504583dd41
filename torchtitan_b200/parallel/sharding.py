"""Declarative sharding contract of a module: where its parameters live on the mesh and how its inputs and
outputs change placement at the module boundary.

Parity: torchtitan/protocols/sharding.py:42-168 (``ShardingConfig`` / ``resolve_placements``) and the per-layer
plans of torchtitan/models/common/decoder_sharding.py:24-376 and moe_sharding.py:40-120.  The reference resolves such a
config into DTensor placements and lets DTensor redistribute; here the same declaration drives three things of the
flat-buffer engine:

* :func:`shard_parameter` cuts the local slice of a parameter out of its full shape from the ``Shard(dim)`` the config
  declares for the axis (and records the slice for initialisation and checkpoints);
* :func:`redistribute` picks the collective for a (source, destination) placement pair on the tensor-parallel axis:
  ``Shard(0) -> Replicate`` all-gathers rows, ``Partial -> Shard(0)`` reduce-scatters rows, ``Partial -> Replicate``
  all-reduces, ``Replicate -> Replicate`` is the identity whose backward sums the gradient;
* :func:`sharding_table` lists the contract of every module of a model, and :func:`check_against_slices` verifies that
  the slices the modules really hold are the ones their contracts declare.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

__all__ = ["Shard", "Replicate", "Partial", "SpmdLayout", "ShardingConfig", "MESH_AXES", "resolve_placements",
           "shard_parameter", "redistribute", "redistribution", "colwise_linear", "rowwise_linear",
           "vocab_parallel_embedding", "sequence_parallel_norm", "expert_tensor_parallel", "expert_parallel",
           "replicated", "sharding_table", "check_against_slices"]

MESH_AXES = ("pp", "dp_replicate", "dp_shard", "cp", "tp", "ep", "efsdp")


@dataclass(frozen=True)
class Shard:
    dim: int

    def __repr__(self):
        return f"S({self.dim})"


@dataclass(frozen=True)
class Replicate:
    def __repr__(self):
        return "R"


@dataclass(frozen=True)
class Partial:
    def __repr__(self):
        return "P"


Placement = Shard | Replicate | Partial


class SpmdLayout(dict):
    """``{mesh axis name: placement}``; axes that are not named are replicated."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        for k in self:
            if k not in MESH_AXES:
                raise ValueError(f"unknown mesh axis '{k}' (known: {MESH_AXES})")

    def on(self, axis: str) -> Placement:
        return self.get(axis, Replicate())


@dataclass(kw_only=True)
class ShardingConfig:
    """``state_shardings``: parameter name -> layout.  ``in_src`` / ``in_dst``: placement of the input named by the
    key before and after the boundary; ``out_src`` / ``out_dst``: the same for the output."""

    state_shardings: dict[str, SpmdLayout] = field(default_factory=dict)
    in_src_shardings: dict[str, SpmdLayout] | None = None
    in_dst_shardings: dict[str, SpmdLayout] | None = None
    out_src_shardings: SpmdLayout | None = None
    out_dst_shardings: SpmdLayout | None = None
    row_blocks: bool = False
    """The sharded dimension is a stack of blocks (``[q | k | v]``, ``[w1 | w3]``), each split evenly."""

    def to_dict(self) -> dict:
        def lay(x):
            return None if x is None else {k: repr(v) for k, v in x.items()}

        return {"state": {k: lay(v) for k, v in self.state_shardings.items()},
                "in": None if self.in_src_shardings is None else
                {k: [lay(v), lay((self.in_dst_shardings or {}).get(k))] for k, v in self.in_src_shardings.items()},
                "out": [lay(self.out_src_shardings), lay(self.out_dst_shardings)]}


def resolve_placements(layout: SpmdLayout, axes: list[tuple[str, int]]) -> tuple[Placement, ...]:
    """Placements in mesh-axis order.  ``Shard`` / ``Partial`` on an axis of size 1 become ``Replicate`` (nothing is
    split and a sum over one rank is the identity)."""
    out = []
    for name, size in axes:
        p = layout.on(name)
        out.append(Replicate() if size == 1 else p)
    return tuple(out)


# ---------------------------------------------------------------------------------------------------------------
# plans


def colwise_linear(sequence_parallel: bool = True, *, blocks: bool = False, bias: bool = False) -> ShardingConfig:
    """Output features split over tp; the input arrives row-sharded (sequence parallel) and is gathered."""
    st = {"weight": SpmdLayout(tp=Shard(0))}
    if bias:
        st["bias"] = SpmdLayout(tp=Shard(0))
    src = SpmdLayout(tp=Shard(0)) if sequence_parallel else SpmdLayout(tp=Replicate())
    return ShardingConfig(state_shardings=st, in_src_shardings={"x": src}, in_dst_shardings={"x": SpmdLayout(tp=Replicate())},
                          out_src_shardings=SpmdLayout(tp=Shard(1)), out_dst_shardings=SpmdLayout(tp=Shard(1)),
                          row_blocks=blocks)


def rowwise_linear(sequence_parallel: bool = True) -> ShardingConfig:
    """Input features split over tp; the output is a partial sum, reduce-scattered to rows or all-reduced."""
    dst = SpmdLayout(tp=Shard(0)) if sequence_parallel else SpmdLayout(tp=Replicate())
    return ShardingConfig(state_shardings={"weight": SpmdLayout(tp=Shard(1))},
                          in_src_shardings={"x": SpmdLayout(tp=Shard(1))}, in_dst_shardings={"x": SpmdLayout(tp=Shard(1))},
                          out_src_shardings=SpmdLayout(tp=Partial()), out_dst_shardings=dst)


def vocab_parallel_embedding(sequence_parallel: bool = True) -> ShardingConfig:
    dst = SpmdLayout(tp=Shard(0)) if sequence_parallel else SpmdLayout(tp=Replicate())
    return ShardingConfig(state_shardings={"weight": SpmdLayout(tp=Shard(0))},
                          in_src_shardings={"tokens": SpmdLayout(tp=Replicate())},
                          in_dst_shardings={"tokens": SpmdLayout(tp=Replicate())},
                          out_src_shardings=SpmdLayout(tp=Partial()), out_dst_shardings=dst)


def sequence_parallel_norm() -> ShardingConfig:
    """Replicated weight on row-sharded activations (its gradient is summed over tp)."""
    lay = SpmdLayout(tp=Shard(0))
    return ShardingConfig(state_shardings={"weight": SpmdLayout(tp=Replicate())}, in_src_shardings={"x": lay},
                          in_dst_shardings={"x": lay}, out_src_shardings=lay, out_dst_shardings=lay)


def replicated(*names: str) -> ShardingConfig:
    return ShardingConfig(state_shardings={n: SpmdLayout(tp=Replicate()) for n in names})


def expert_tensor_parallel(sequence_parallel: bool = True) -> ShardingConfig:
    """Experts ``[E, out, in]`` without expert parallelism: w1 / w3 split over their output (hidden) dimension, w2
    over its input; tokens are gathered over tp and the layer's output is a partial sum."""
    src = SpmdLayout(tp=Shard(0)) if sequence_parallel else SpmdLayout(tp=Replicate())
    return ShardingConfig(state_shardings={"w1_EFD": SpmdLayout(tp=Shard(1)), "w3_EFD": SpmdLayout(tp=Shard(1)),
                                           "w2_EDF": SpmdLayout(tp=Shard(2))},
                          in_src_shardings={"x": src}, in_dst_shardings={"x": SpmdLayout(tp=Replicate())},
                          out_src_shardings=SpmdLayout(tp=Partial()), out_dst_shardings=src)


def expert_parallel() -> ShardingConfig:
    """Experts split over ep along the expert dimension; parameters are then sharded over efsdp by the engine."""
    lay = SpmdLayout(ep=Shard(0))
    return ShardingConfig(state_shardings={"w1_EFD": lay, "w2_EDF": lay, "w3_EFD": lay})


# ---------------------------------------------------------------------------------------------------------------
# the contract applied


def _even_slices(blocks: list[int], size: int, rank: int) -> list[tuple[int, int]]:
    out, base = [], 0
    for b in blocks:
        if b % size:
            raise ValueError(f"a block of {b} is not divisible by the axis size {size}")
        step = b // size
        out.append((base + rank * step, base + (rank + 1) * step))
        base += b
    return out


def shard_parameter(param: nn.Parameter, placement: Placement, size: int, rank: int, *, blocks: list[int] | None = None,
                    full_shape: tuple[int, ...] | None = None) -> nn.Parameter:
    """The local part of ``param`` (meta device or real) under ``placement`` on an axis of ``size`` ranks: a new
    parameter of the sliced shape that remembers ``(dim, ranges, full shape)`` in ``_tp_slices`` and keeps the
    initialisation spec.  ``Replicate`` returns ``param`` itself, marked as replicated over the axis."""
    from torchtitan_b200.models.common.module import set_init

    if isinstance(placement, Partial):
        raise ValueError("a parameter cannot be Partial")
    if isinstance(placement, Replicate):
        param._replicated_over_tp = True
        return param
    dim = placement.dim
    shape = tuple(param.shape)
    ranges = _even_slices(blocks or [shape[dim]], size, rank)
    n = sum(b - a for a, b in ranges)
    new_shape = shape[:dim] + (n,) + shape[dim + 1:]
    new = nn.Parameter(torch.empty(new_shape, device=param.device, dtype=param.dtype), requires_grad=param.requires_grad)
    new._tp_slices = (dim, ranges, tuple(full_shape or shape))
    if hasattr(param, "_init_spec"):
        set_init(new, param._init_spec)
    return new


def redistribution(src: Placement, dst: Placement) -> str:
    """Name of the collective that turns ``src`` into ``dst`` on one axis."""
    if isinstance(src, Partial):
        if isinstance(dst, Shard):
            if dst.dim != 0:
                raise ValueError("partial sums are reduce-scattered over rows (dim 0) only")
            return "reduce_scatter_rows"
        if isinstance(dst, Replicate):
            return "all_reduce"
        return "none"
    if isinstance(src, Shard):
        if isinstance(dst, Replicate):
            if src.dim != 0:
                raise ValueError("only row-sharded activations are gathered")
            return "all_gather_rows"
        if dst == src:
            return "none"
        raise ValueError(f"no collective for {src!r} -> {dst!r}")
    if isinstance(dst, Replicate):
        return "copy"  # identity; the backward sums the gradient over the axis
    if isinstance(dst, Shard):
        return "slice"
    raise ValueError(f"no collective for {src!r} -> {dst!r}")


def redistribute(x: torch.Tensor, src: Placement, dst: Placement, tp) -> torch.Tensor:
    """Apply :func:`redistribution` on the tensor-parallel axis (autograd-aware collectives of ``tp_ops``)."""
    from . import tp_ops

    kind = redistribution(src, dst)
    if kind == "none" or tp is None or tp.size == 1:
        return x
    if kind == "all_gather_rows":
        return tp_ops.all_gather_rows(x, tp)
    if kind == "reduce_scatter_rows":
        return tp_ops.reduce_scatter_rows(x, tp)
    if kind == "all_reduce":
        return tp_ops.all_reduce(x, tp)
    if kind == "copy":
        return tp_ops.copy_to_tp(x, tp)
    n = x.shape[dst.dim] // tp.size
    return x.narrow(dst.dim, tp.rank * n, n)


# ---------------------------------------------------------------------------------------------------------------
# inspection


def sharding_table(model: nn.Module) -> dict[str, dict]:
    """``{module path: contract}`` for every module that declared one."""
    return {name: m.sharding.to_dict() for name, m in model.named_modules() if getattr(m, "sharding", None) is not None}


def check_against_slices(model: nn.Module, axis: str = "tp") -> int:
    """Every parameter whose module declares ``Shard(d)`` on ``axis`` must hold a slice of dimension ``d``; every
    parameter declared ``Replicate`` must hold none.  Returns the number of parameters checked."""
    n = 0
    for mod_name, m in model.named_modules():
        cfg = getattr(m, "sharding", None)
        if cfg is None:
            continue
        for pname, layout in cfg.state_shardings.items():
            p = getattr(m, pname, None)
            if p is None:
                continue
            placement = layout.on(axis)
            held = getattr(p, "_tp_slices", None)
            if isinstance(placement, Shard):
                if held is None or held[0] != placement.dim:
                    raise RuntimeError(f"{mod_name}.{pname}: declared {placement!r} on {axis}, holds {held}")
            elif axis in layout and held is not None:
                raise RuntimeError(f"{mod_name}.{pname}: declared replicated on {axis}, holds the slice {held}")
            n += 1
    return n
