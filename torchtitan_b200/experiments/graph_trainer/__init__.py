"""graph_trainer: the user-facing surface of the reference's graph-based trainer on this framework's mechanisms.

The reference (torchtitan/experiments/graph_trainer) traces the whole training step into an FX graph and applies
passes to it: FSDP bucketing and overlap reordering (fsdp_passes.py), async tensor parallelism (passes.py:95-131),
expert-parallel chunk / overlap passes, selective rematerialisation and CPU activation offload (memory_policy.py,
cpu_offload.py), CUDA graphs (cudagraph.py) and ahead-of-time compilation on one rank (precompile.py).  This
framework has no tracing compiler by design: what those passes *achieve* exists here as properties of the engine
and of hand-written kernels.  ``GraphTrainer`` keeps the reference's way of asking for them: a list of pass names
in ``compile.passes``, which ``apply_passes`` turns into the corresponding settings:

====================  =========================================================================================
pass                  what it switches on here
====================  =========================================================================================
``cudagraph``         forward + backward replayed from a CUDA graph (``parallel/cudagraph.py``)
``fsdp_overlap``      reduce-scatter per unit under the backward, optimizer + weight refresh under the next
                      forward (always on in the engine; ``TB200_OVERLAP_OPTIMIZER=0`` is the off switch)
``fsdp_reshard``      sharded parameter layout with one-unit-ahead prefetch (``fsdp_reshard_after_forward=always``)
``async_tp``          all-gather -> GEMM and GEMM -> reduce-scatter in one kernel each (``tp_comm = nvlink``)
``ep_overlap``        sync-free expert-parallel dispatch over NVLink (``ep_comm = nvlink``)
``cpu_offload``       activations offloaded to pinned host memory on a side stream
``selective_remat``   selective activation recomputation (norm / SwiGLU recomputed, GEMM outputs kept)
``full_remat``        full activation checkpointing
``precompile``        the sm_100a extension is built once by rank 0 before training (the ahead-of-time artifact
                      is the shared object under ``ops/_build``), all ranks load it
``regional_inductor`` accepted and ignored with a warning: there is no Inductor path
``full_inductor``     accepted and ignored with a warning
====================  =========================================================================================
"""

from __future__ import annotations

from torchtitan_b200.trainer import Trainer
from torchtitan_b200.utils.logging import logger

__all__ = ["GraphTrainer", "apply_passes", "KNOWN_PASSES", "precompile"]

KNOWN_PASSES = ("cudagraph", "fsdp_overlap", "fsdp_reshard", "async_tp", "ep_overlap", "cpu_offload", "selective_remat",
                "full_remat", "precompile", "regional_inductor", "full_inductor")


def apply_passes(config: "Trainer.Config", passes: list[str], *, run_precompile: bool = True) -> list[str]:
    """Fold the pass list into ``config`` (in place); returns the passes that changed something.  With
    ``run_precompile=False`` the ``precompile`` pass is only recorded (the caller builds once the process group is
    up, so that rank 0 builds and the others wait)."""
    done = []
    for name in passes:
        if name not in KNOWN_PASSES:
            raise ValueError(f"unknown graph_trainer pass '{name}'; known: {', '.join(KNOWN_PASSES)}")
        if name == "cudagraph":
            config.training.disable_cuda_graphs = False
        elif name == "fsdp_reshard":
            config.parallelism.fsdp_reshard_after_forward = "always"
        elif name == "async_tp":
            config.parallelism.tp_comm = "nvlink"
        elif name == "ep_overlap":
            config.parallelism.ep_comm = "nvlink"
        elif name == "cpu_offload":
            config.activation_checkpoint.cpu_offload = True
        elif name == "selective_remat":
            config.activation_checkpoint.mode = "selective"
        elif name == "full_remat":
            config.activation_checkpoint.mode = "full"
        elif name == "precompile":
            if run_precompile:
                precompile()
        elif name in ("regional_inductor", "full_inductor"):
            logger.warning(f"graph_trainer pass '{name}' is accepted for compatibility: this framework runs hand-written "
                           "kernels, there is no Inductor path")
            continue
        done.append(name)
    if "cudagraph" in done and "cpu_offload" in done:
        raise ValueError("cudagraph and cpu_offload cannot be combined: host copies cannot be captured")
    return done


def precompile() -> None:
    """Build the extension on rank 0 (if stale), then let everybody load the same shared object."""
    import torch.distributed as dist

    from torchtitan_b200.ops import ext

    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        ext.build()
    if dist.is_initialized():
        dist.barrier()
    ext.load()


class GraphTrainer(Trainer):
    """``Trainer`` whose config carries ``compile.passes``-style requests (see the module docstring)."""

    def __init__(self, config: "Trainer.Config", *, passes: list[str] | None = None, **kw):
        self.applied_passes = apply_passes(config, list(passes or []))
        if self.applied_passes:
            logger.info(f"graph_trainer passes: {self.applied_passes}")
        super().__init__(config, **kw)
