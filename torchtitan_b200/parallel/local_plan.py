"""``comm.mode = "local_tensor"``: one process plays every rank of an ``NGPU``-rank job, one after the other, and
checks the parallel plan without running a single collective or allocating a parameter.

For each rank the model is built on the meta device, the tensor / expert / pipeline slicing and the sharded
data-parallel units are derived exactly as the real job would (``parallelize_fn(..., materialize=False)``), and the
pieces of every parameter that the rank would own are recorded.  At the end every parameter of the model must be
covered exactly once per data-parallel replica: no element missing, none owned twice.  The reference offers the
same dry run through LocalTensor (torchtitan/train.py:47-49, torchtitan/distributed/utils.py:448-452), also
returning before training."""

from __future__ import annotations

import os
from collections import defaultdict

import torch
import torch.distributed as dist

from torchtitan_b200.utils.logging import logger

__all__ = ["validate_plan"]


def _rank_plan(config, world: int, rank: int) -> tuple[dict[str, int], dict[str, int]]:
    """``({fqn: elements owned by this rank}, {fqn: global numel})`` for one emulated rank."""
    from torch.testing._internal.distributed.fake_pg import FakeStore

    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.parallel.parallel_dims import ParallelDims

    dist.init_process_group("fake", rank=rank, world_size=world, store=FakeStore())
    try:
        pdims = ParallelDims.from_config(config.parallelism, world, rank).build()
        spec = config.model_spec or get_model_spec(config.model.name, config.model.flavor)
        model_cfg = spec.model
        model_cfg.update_from_config(trainer_config=config)
        with torch.device("meta"):
            model = model_cfg.build()
        if pdims.pp_enabled:
            raise NotImplementedError("plan validation covers one pipeline stage layout per job; run it with pp = 1")
        engine = spec.parallelize_fn(model, pdims=pdims, job_config=config, device=torch.device("meta"), seed=0,
                                     grad_accum_steps=1, materialize=False)
        owned: dict[str, int] = defaultdict(int)
        total: dict[str, int] = {}
        for u in engine.units:
            for slot in u.slots:
                g = 1
                for d in (slot.tp_slices[2] if slot.tp_slices is not None else slot.shape):
                    g *= d
                total[slot.fqn] = g
            for slot, _pstart, _sstart, n in u.slot_pieces():
                owned[slot.fqn] += n
        replicas = {}
        for u in engine.units:
            for slot in u.slots:
                # ranks that hold the same elements: the replicate axis, and tensor-parallel ranks for replicated parameters
                r = max(1, pdims.dp_replicate)
                if slot.tp_slices is None and pdims.tp_enabled:
                    r *= pdims.tp
                replicas[slot.fqn] = r
        return dict(owned), {k: v * replicas[k] for k, v in total.items()}
    finally:
        dist.destroy_process_group()


def validate_plan(config, world: int | None = None) -> dict[str, int]:
    """Raises if the ranks' shards do not tile the parameters; returns ``{fqn: numel}`` of the covered parameters."""
    world = world or int(os.environ.get("NGPU", os.environ.get("WORLD_SIZE", "1")))
    if dist.is_initialized():
        raise RuntimeError("local_tensor mode builds its own (fake) process groups; start it from a plain process")
    covered: dict[str, int] = defaultdict(int)
    expected: dict[str, int] = {}
    for rank in range(world):
        owned, total = _rank_plan(config, world, rank)
        for k, v in owned.items():
            covered[k] += v
        for k, v in total.items():
            expected[k] = max(expected.get(k, 0), v)
    bad = {k: (covered.get(k, 0), v) for k, v in expected.items() if covered.get(k, 0) != v}
    if bad:
        some = ", ".join(f"{k}: covered {c} of {v}" for k, (c, v) in list(bad.items())[:5])
        raise RuntimeError(f"the parallel plan does not tile {len(bad)} parameter(s) exactly once: {some}")
    logger.info(f"local_tensor: {world} emulated ranks tile {len(expected)} parameters "
                f"({sum(expected.values()):,} elements including replicas) exactly once")
    return dict(expected)
