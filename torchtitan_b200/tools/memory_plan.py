"""Per-GPU memory plan of a job, computed on the meta device (nothing is allocated, no process group is needed):

    python -m torchtitan_b200.tools.memory_plan --module llama3 --config llama3_405b --world 512 \\
        --parallelism.tensor_parallel_degree 8 --parallelism.pipeline_parallel_degree 1

For one rank the model is built on the meta device and parallelised exactly like the real job
(``materialize=False``); the plan then adds up what the sharded engine would hold: parameter and gradient buffers
of the chosen layout (resident: full-size per unit; sharded: the rank's shards plus two gather slots and two
gradient slots per group), fp32 master weights, the fp32 gradient shards and both optimizer moments.  Activations
are not modelled (they depend on the recomputation mode and the sequence length); ``fits`` compares the static
part against a budget.  Counterpart of the reference's memory estimation tool (scripts/estimate/estimation.py)."""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

__all__ = ["MemoryPlan", "plan_memory"]

GiB = float(1 << 30)


@dataclass
class MemoryPlan:
    layout: str
    params_gib: float
    grads_gib: float
    grad_shards_gib: float
    master_gib: float
    moments_gib: float
    largest_unit_gib: float
    local_params: int

    @property
    def total_gib(self) -> float:
        return self.params_gib + self.grads_gib + self.grad_shards_gib + self.master_gib + self.moments_gib

    def fits(self, budget_gib: float = 180.0, activation_reserve_gib: float = 40.0) -> bool:
        return self.total_gib + activation_reserve_gib <= budget_gib

    def __str__(self) -> str:
        return (f"{self.layout}: parameters {self.params_gib:.1f} GiB, gradient buffers {self.grads_gib:.1f}, fp32 gradient "
                f"shards {self.grad_shards_gib:.1f}, fp32 master {self.master_gib:.1f}, moments {self.moments_gib:.1f} "
                f"-> {self.total_gib:.1f} GiB per GPU ({self.local_params:,} parameters on this rank before data-parallel "
                f"sharding, largest unit {self.largest_unit_gib:.2f} GiB)")


def plan_memory(config, world: int, rank: int = 0, *, param_bytes: int = 2, state_bytes: int | None = None) -> MemoryPlan:
    from torch.testing._internal.distributed.fake_pg import FakeStore

    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.parallel.parallel_dims import ParallelDims

    if dist.is_initialized():
        raise RuntimeError("plan_memory builds its own (fake) process group; call it from a plain process")
    if state_bytes is None:
        state_bytes = 2 if getattr(config.optimizer, "implementation", "fused") == "fused_opt_states_bf16" else 4
    dist.init_process_group("fake", rank=rank, world_size=world, store=FakeStore())
    try:
        pdims = ParallelDims.from_config(config.parallelism, world, rank).build()
        spec = config.model_spec or get_model_spec(config.model.name, config.model.flavor)
        model_cfg = spec.model
        model_cfg.update_from_config(trainer_config=config)
        with torch.device("meta"):
            model = model_cfg.build()
        if pdims.pp_enabled:
            # a pipeline rank holds 1 / pp of the blocks (embedding / head on the end stages are ignored here)
            keep = max(1, len(model.layers) // pdims.pp)
            for name in list(model.layers.keys())[keep:]:
                del model.layers[name]
        engine = spec.parallelize_fn(model, pdims=pdims, job_config=config, device=torch.device("meta"), seed=0,
                                     grad_accum_steps=2, materialize=False)
        policy = config.parallelism.fsdp_reshard_after_forward
        multi = [u for u in engine.units if u.size > 1]
        replicated = sum(2 * u.padded * param_bytes for u in multi)
        sharded = bool(multi) and (policy == "always" or (policy == "default" and replicated > 180 * GiB / 3))
        params = grads = 0.0
        biggest: dict[int, int] = {}
        for u in engine.units:
            if sharded and u.size > 1:
                params += u.shard_numel * param_bytes
                biggest[id(u.group)] = max(biggest.get(id(u.group), 0), u.padded)
            else:
                params += u.padded * param_bytes
                grads += u.padded * param_bytes
        for n in biggest.values():
            params += 2 * n * param_bytes
            grads += 2 * n * param_bytes
        shard_elems = sum(u.shard_numel for u in engine.units)
        return MemoryPlan(
            layout="sharded parameters" if sharded else "resident parameters",
            params_gib=params / GiB, grads_gib=grads / GiB, grad_shards_gib=shard_elems * 4 / GiB,
            master_gib=shard_elems * 4 / GiB, moments_gib=2 * shard_elems * state_bytes / GiB,
            largest_unit_gib=max(u.padded for u in engine.units) * param_bytes / GiB,
            local_params=sum(u.numel for u in engine.units))
    finally:
        dist.destroy_process_group()


def main(argv=None) -> None:
    import argparse

    from torchtitan_b200.config import ConfigManager

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--world", type=int, default=int(os.environ.get("NGPU", "8")))
    args, rest = ap.parse_known_args(argv)
    config = ConfigManager().parse_args(rest)
    plan = plan_memory(config, args.world)
    print(plan)
    print("fits in 180 GB with 40 GiB kept for activations:", plan.fits())


if __name__ == "__main__":
    main()
