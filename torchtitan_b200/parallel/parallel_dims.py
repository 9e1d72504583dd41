"""Rank grid and process groups for N-D parallelism.

The world is a dense grid ``[pp, dp_replicate, dp_shard, cp, tp]`` with ``tp``
varying fastest, so tensor-parallel peers are neighbouring ranks (on one
NVSwitch domain that choice is bandwidth-neutral, it only keeps the rank maths
the same as the reference).  Expert parallelism borrows the ranks of
``dp_shard x cp x tp``: ``ep`` must divide that product and the remaining factor
is ``efsdp``, the axis expert parameters are sharded over.

Named axes (each resolvable to a process group through :meth:`group`):

``pp dp_replicate dp_shard cp tp``  the five base axes
``dp``      dp_replicate x dp_shard         (data loading: distinct batches)
``batch``   same ranks as ``dp``            (valid-token count)
``fsdp``    dp_shard x cp                   (parameter sharding of dense weights)
``loss``    dp_replicate x dp_shard x cp    (loss / metric reduction)
``ep``, ``efsdp``                           (sparse weights)

Parity: torchtitan/distributed/parallel_dims.py:132-671.  Groups of size one are
never created; ``group`` returns ``None`` for them and callers skip the
collective.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterable

import torch
import torch.distributed as dist

__all__ = ["ParallelDims", "BASE_AXES"]

BASE_AXES = ("pp", "dp_replicate", "dp_shard", "cp", "tp")

_DERIVED = {
    "dp": ("dp_replicate", "dp_shard"),
    "batch": ("dp_replicate", "dp_shard"),
    "fsdp": ("dp_shard", "cp"),
    "dp_shard_cp": ("dp_shard", "cp"),
    "loss": ("dp_replicate", "dp_shard", "cp"),
    "dp_cp": ("dp_replicate", "dp_shard", "cp"),
}


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    world_size: int = 1
    rank: int = 0
    _groups: dict[str, Any] = field(default_factory=dict, repr=False)
    _built: bool = field(default=False, repr=False)

    # ------------------------------------------------------------------
    @classmethod
    def from_config(cls, parallelism, world_size: int, rank: int = 0) -> "ParallelDims":
        return cls(
            dp_replicate=parallelism.data_parallel_replicate_degree,
            dp_shard=parallelism.data_parallel_shard_degree,
            cp=parallelism.context_parallel_degree,
            tp=parallelism.tensor_parallel_degree,
            pp=parallelism.pipeline_parallel_degree,
            ep=parallelism.expert_parallel_degree,
            world_size=world_size,
            rank=rank,
        )

    def __post_init__(self):
        for name in ("dp_replicate", "cp", "tp", "pp", "ep"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} degree must be >= 1, got {getattr(self, name)}")
        if self.dp_shard != -1 and self.dp_shard < 1:
            raise ValueError("dp_shard degree must be -1 or >= 1")
        rest = self.dp_replicate * self.cp * self.tp * self.pp
        if self.dp_shard == -1:
            if self.world_size % rest:
                raise ValueError(
                    f"world size {self.world_size} is not divisible by dp_replicate*cp*tp*pp = {rest}"
                )
            self.dp_shard = self.world_size // rest
        if self.dp_shard * rest != self.world_size:
            raise ValueError(
                f"dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * "
                f"tp({self.tp}) * pp({self.pp}) != world size {self.world_size}"
            )
        if self.ep > 1:
            pool = self.dp_shard * self.cp * self.tp
            if pool % self.ep:
                raise ValueError(f"ep({self.ep}) must divide dp_shard*cp*tp = {pool}")
        if not 0 <= self.rank < self.world_size:
            raise ValueError("rank out of range")

    # ------------------------------------------------------------------
    @property
    def shape(self) -> tuple[int, ...]:
        return (self.pp, self.dp_replicate, self.dp_shard, self.cp, self.tp)

    @property
    def efsdp(self) -> int:
        return self.dp_shard * self.cp * self.tp // self.ep

    def coords(self, rank: int | None = None) -> dict[str, int]:
        r = self.rank if rank is None else rank
        out = {}
        for name, size in zip(reversed(BASE_AXES), reversed(self.shape)):
            out[name] = r % size
            r //= size
        return out

    def rank_of(self, **coords: int) -> int:
        r = 0
        for name, size in zip(BASE_AXES, self.shape):
            r = r * size + coords[name]
        return r

    def _axes_of(self, name: str) -> tuple[str, ...]:
        if name in BASE_AXES:
            return (name,)
        if name in _DERIVED:
            return _DERIVED[name]
        raise KeyError(f"unknown mesh axis '{name}'")

    def size(self, name: str) -> int:
        if name == "ep":
            return self.ep
        if name == "efsdp":
            return self.efsdp
        if name == "world":
            return self.world_size
        n = 1
        for a in self._axes_of(name):
            n *= getattr(self, a)
        return n

    def ranks_in(self, name: str, rank: int | None = None) -> list[int]:
        """World ranks of the ``name`` group that contains ``rank`` (ordered)."""
        me = self.coords(rank)
        if name == "world":
            return list(range(self.world_size))
        if name in ("ep", "efsdp"):
            # The sparse pool is the flattened (dp_shard, cp, tp) index; ep varies fastest.
            pool_axes = ("dp_shard", "cp", "tp")
            sizes = [getattr(self, a) for a in pool_axes]
            flat = 0
            for a, s in zip(pool_axes, sizes):
                flat = flat * s + me[a]
            ep_idx, ef_idx = flat % self.ep, flat // self.ep
            out = []
            n = self.ep if name == "ep" else self.efsdp
            for i in range(n):
                f = (ef_idx * self.ep + i) if name == "ep" else (i * self.ep + ep_idx)
                c = dict(me)
                for a, s in zip(reversed(pool_axes), reversed(sizes)):
                    c[a] = f % s
                    f //= s
                out.append(self.rank_of(**c))
            return out
        axes = self._axes_of(name)
        out = [dict(me)]
        for a in axes:
            out = [dict(c, **{a: i}) for c in out for i in range(getattr(self, a))]
        return [self.rank_of(**c) for c in out]

    def local_rank(self, name: str) -> int:
        return self.ranks_in(name).index(self.rank)

    # ------------------------------------------------------------------
    def build(self) -> "ParallelDims":
        """Create every process group with more than one member.

        ``new_group`` is collective over the world, so all ranks enumerate the
        same partitions in the same order.
        """
        if self._built:
            return self
        self._built = True
        if not dist.is_initialized() or self.world_size == 1:
            return self
        names = list(BASE_AXES) + ["dp", "fsdp", "loss", "ep", "efsdp"]
        made: dict[tuple[int, ...], Any] = {}
        for name in names:
            if self.size(name) == 1:
                continue
            seen: set[tuple[int, ...]] = set()
            for r in range(self.world_size):
                ranks = tuple(self.ranks_in(name, r))
                if ranks in seen:
                    continue
                seen.add(ranks)
                if ranks not in made:
                    made[ranks] = dist.group.WORLD if len(ranks) == self.world_size and list(ranks) == list(range(self.world_size)) else dist.new_group(list(ranks))
                if self.rank in ranks:
                    self._groups[name] = made[ranks]
        for alias, target in (("batch", "dp"), ("dp_shard_cp", "fsdp"), ("dp_cp", "loss")):
            if target in self._groups:
                self._groups[alias] = self._groups[target]
        return self

    def group(self, name: str):
        """Process group of axis ``name`` or ``None`` when its size is one."""
        if self.size(name) == 1:
            return None
        if name == "world":
            return dist.group.WORLD
        if not self._built:
            self.build()
        return self._groups.get(name)

    def device_mesh(self, name: str, device_type: str):
        """1-D ``DeviceMesh`` over axis ``name`` (used for DTensor checkpoint metadata)."""
        from torch.distributed.device_mesh import DeviceMesh

        g = self.group(name)
        if g is None:
            return None
        return DeviceMesh.from_group(g, device_type, mesh=self.ranks_in(name), mesh_dim_names=(name,))

    # ------------------------------------------------------------------
    dp_enabled = property(lambda s: s.dp_replicate * s.dp_shard > 1)
    dp_replicate_enabled = property(lambda s: s.dp_replicate > 1)
    dp_shard_enabled = property(lambda s: s.dp_shard > 1)
    cp_enabled = property(lambda s: s.cp > 1)
    dp_cp_enabled = property(lambda s: s.dp_enabled or s.cp_enabled)
    fsdp_enabled = property(lambda s: s.dp_shard_enabled or s.cp_enabled)
    tp_enabled = property(lambda s: s.tp > 1)
    pp_enabled = property(lambda s: s.pp > 1)
    ep_enabled = property(lambda s: s.ep > 1)

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp * self.pp

    @property
    def seq_len_divisor(self) -> int:
        """Token counts must divide by this (SP shards by tp, CP by 2*cp chunks)."""
        return self.tp * (2 * self.cp if self.cp > 1 else 1)

    @property
    def dp_degree(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def dp_rank(self) -> int:
        c = self.coords()
        return c["dp_replicate"] * self.dp_shard + c["dp_shard"]
