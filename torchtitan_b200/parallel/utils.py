"""Process-group bootstrap, determinism, scalar reductions, timeouts.

Parity: torchtitan/distributed/utils.py:98-740.  One process per GPU; NCCL for
CUDA tensors, gloo for CPU tensors (both are registered so checkpoint planning and
CPU tests use the same code).  Environment for the NCCL flight recorder is set
before the process group exists.
"""

from __future__ import annotations

import os
from datetime import timedelta

import torch
import torch.distributed as dist

from torchtitan_b200.utils.logging import logger

__all__ = ["pin_nccl_for_batch_invariance", "init_distributed", "set_determinism", "dist_sum", "dist_max", "dist_mean", "dist_min",
           "set_pg_timeouts", "destroy", "world_info"]


def pin_nccl_for_batch_invariance() -> dict[str, str]:
    """Fix every NCCL choice that may depend on load or message size, so that reductions add in one order (must run
    before the process group is created; values already present in the environment win).  Parity:
    torchtitan/distributed/utils.py:345-370."""
    pins = {
        "NCCL_LAUNCH_MODE": "GROUP", "NCCL_COLLNET_ENABLE": "0", "NCCL_NVLS_ENABLE": "0", "NCCL_P2P_NET_DISABLE": "1",
        "NCCL_MIN_NCHANNELS": "4", "NCCL_MAX_NCHANNELS": "4", "NCCL_PROTO": "Simple", "NCCL_ALGO": "Ring",
        "NCCL_NTHREADS": "512",
    }
    applied = {}
    for k, v in pins.items():
        if k not in os.environ:
            os.environ[k] = v
            applied[k] = v
    return applied


def world_info() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init_distributed(comm_config, device: torch.device, *, dump_folder: str = "./outputs",
                     enable_cpu_backend: bool = False) -> int:
    """Initialise the default process group when launched with more than one rank."""
    rank, _, world = world_info()
    if dist.is_initialized():  # embedded use (tests, notebooks): keep the caller's process group
        return dist.get_world_size()
    mode = getattr(comm_config, "mode", "default")
    if mode == "fake_backend":
        from torch.testing._internal.distributed.fake_pg import FakeStore

        world = int(os.environ.get("NGPU", os.environ.get("WORLD_SIZE", "1")))
        dist.init_process_group("fake", rank=rank, world_size=world, store=FakeStore())
        return world
    if mode == "torchcomms":
        logger.warning("comm.mode = torchcomms: the torchcomms package is not part of this build; using the default "
                       "torch.distributed process groups (NCCL / gloo)")
    if world == 1 and "MASTER_ADDR" not in os.environ:
        return 1

    def _set(name: str, value: str) -> None:
        if name not in os.environ:
            os.environ[name] = value

    # NCCL watchdog / flight recorder (dump per-rank traces when a collective times out)
    _set("TORCH_NCCL_ASYNC_ERROR_HANDLING", "3")
    _set("TORCH_FR_BUFFER_SIZE", str(comm_config.trace_buf_size))
    if comm_config.trace_buf_size > 0:
        trace_dir = os.path.join(dump_folder, comm_config.save_traces_folder)
        os.makedirs(trace_dir, exist_ok=True)
        _set("TORCH_NCCL_DUMP_ON_TIMEOUT", "1")
        _set("TORCH_FR_DUMP_TEMP_FILE", os.path.join(trace_dir, comm_config.save_traces_file_prefix))
    if device.type == "cuda":
        backend = "cuda:nccl,cpu:gloo"
    else:
        backend = "gloo"
    kw = {}
    if device.type == "cuda":
        kw["device_id"] = device
    dist.init_process_group(backend=backend, timeout=timedelta(seconds=comm_config.init_timeout_seconds), **kw)
    torch.autograd.set_multithreading_enabled(False)
    return dist.get_world_size()


def set_determinism(pdims, device: torch.device, seed: int | None, deterministic: bool = False,
                    warn_only: bool = False, distinct_seed_axes: tuple[str, ...] = ("pp",)) -> int:
    """Seed all RNGs.  Ranks agree on the base seed (rank 0's when none is given);
    ranks that differ along ``distinct_seed_axes`` get different streams (dropout,
    data noise), everything else is identical.  Parameter init does not depend on
    these streams."""
    if deterministic:
        logger.info("Deterministic algorithms enabled")
        torch.use_deterministic_algorithms(True, warn_only=warn_only)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    if seed is None:
        t = torch.get_rng_state()[:8].to(device) if device.type != "cpu" else torch.get_rng_state()[:8].clone()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.broadcast(t, src=0)
        seed = int(t.cpu().view(torch.uint64).item() % (1 << 62))
    offset = 0
    if pdims is not None:
        c = pdims.coords()
        mul = 1
        for ax in distinct_seed_axes:
            offset += c.get(ax, 0) * mul
            mul *= max(1, pdims.size(ax))
    torch.manual_seed((seed + offset) % (1 << 63))
    os.environ["PYTHONHASHSEED"] = str((seed + offset) % (1 << 32))
    return seed


def _reduce(x, op, group):
    if isinstance(x, torch.Tensor):
        t = x.detach().clone().reshape(1)
    else:
        t = torch.tensor([float(x)])
    if group is not None and dist.is_initialized():
        dist.all_reduce(t, op=op, group=group)
    return t


def dist_sum(x, group) -> float:
    return _reduce(x, dist.ReduceOp.SUM, group).item()


def dist_max(x, group) -> float:
    return _reduce(x, dist.ReduceOp.MAX, group).item()


def dist_min(x, group) -> float:
    return _reduce(x, dist.ReduceOp.MIN, group).item()


def dist_mean(x, group) -> float:
    n = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    return _reduce(x, dist.ReduceOp.SUM, group).item() / n


def set_pg_timeouts(timeout_seconds: int, pdims) -> None:
    """Tighten collective timeouts after the first step (lazy init and warm-up are over)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return
    logger.info(f"Synchronizing and adjusting timeout for all ProcessGroups to {timeout_seconds}s")
    dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    groups = [dist.group.WORLD] + [g for g in getattr(pdims, "_groups", {}).values() if g is not None]
    seen = set()
    set_timeout = getattr(dist.distributed_c10d, "_set_pg_timeout", None)
    for g in groups:
        if id(g) in seen or set_timeout is None:
            continue
        seen.add(id(g))
        try:
            set_timeout(timedelta(seconds=timeout_seconds), g)
        except Exception as e:  # gloo groups may not support it
            logger.debug(f"could not set timeout on {g}: {e}")


def destroy() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
