"""Fault-tolerant replicated training on top of the regular trainer (parity:
torchtitan/experiments/torchft/{trainer,optimizer,checkpoint}.py and config/job_config.py).

Every *replica group* is an ordinary job of this framework (its own ``torch.distributed`` world with any
FSDP / TP / PP layout).  Replica groups are tied together only through the ``FTManager`` store:

* ``FTOptimizersContainer``: ``zero_grad`` opens the step's quorum (who is alive and takes part), ``step`` applies
  the update only if the step can be committed (no member was lost while gradients were averaged);
* ``FaultTolerantTrainer``: after the in-group reduce-scatter each rank averages its gradient shards with the same
  rank of the other live replicas (``FTManager.allreduce``; the loss the trainer divides by counts the tokens of
  the participating replicas); with ``semi_sync_method`` = ``local_sgd`` / ``diloco`` gradients stay local and the
  parameters (or pseudo-gradients) are averaged every ``sync_steps`` steps instead;
* ``FTCheckpointManager``: besides the regular checkpoints every replica writes its own data-loader position each
  step (``ft-replica-<id>/``), so that a restarted replica resumes its own data stream while the model state comes
  from a live replica's checkpoint.

A replica leaves only between steps and is noticed on the host through its heartbeat; no device-side wait is
involved.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta

import torch

from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.trainer import Trainer
from torchtitan_b200.utils.logging import logger

from .manager import FTManager
from .semi_sync import DiLoCo, LocalSGD

__all__ = ["FaultToleranceConfig", "FTOptimizersContainer", "FTCheckpointManager", "FaultTolerantTrainer", "fragment_llm"]


@dataclass(kw_only=True, slots=True)
class FaultToleranceConfig:
    enable: bool = False
    replica_id: int = 0
    group_size: int = 1            # number of replica groups
    min_replica_size: int = 1
    store_addr: str = "127.0.0.1"
    store_port: int = 29600
    heartbeat_timeout_s: float = 5.0
    quorum_timeout_s: float = 30.0
    semi_sync_method: str | None = None      # None | "local_sgd" | "diloco"
    sync_steps: int = 5
    num_fragments: int = 1                   # DiLoCo: parameters are split into this many fragments (by blocks)


class FTOptimizersContainer:
    """Wraps the regular container: quorum at ``zero_grad``, commit check at ``step``."""

    def __init__(self, inner: OptimizersContainer, manager: FTManager):
        self.inner, self.manager = inner, manager
        self._step = 0
        self.skipped = 0

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.manager.start_quorum(self._step)
        self.inner.zero_grad(set_to_none)

    def step(self) -> None:
        self._step += 1
        if self.manager.should_commit():
            self.inner.step()
        else:
            self.skipped += 1
            logger.warning(f"fault tolerance: step {self._step} not committed (a replica left during the average)")


class FTCheckpointManager:
    """Per-replica data-loader checkpoints next to the regular checkpoint manager (whose calls pass through)."""

    def __init__(self, inner, dataloader, replica_id: int, dump_folder: str):
        self.inner, self.dataloader = inner, dataloader
        self.folder = os.path.join(dump_folder, f"ft-replica-{replica_id}")
        os.makedirs(self.folder, exist_ok=True)

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def save(self, step: int, last_step: bool = False) -> None:
        sd = self.dataloader.state_dict() if hasattr(self.dataloader, "state_dict") else {}
        tmp = os.path.join(self.folder, "dataloader.tmp")
        torch.save({"step": step, "dataloader": sd}, tmp)
        os.replace(tmp, os.path.join(self.folder, "dataloader.pt"))
        self.inner.save(step, last_step=last_step)

    def load(self, step: int = -1) -> bool:
        ok = self.inner.load(step=step)
        path = os.path.join(self.folder, "dataloader.pt")
        if os.path.exists(path) and hasattr(self.dataloader, "load_state_dict"):
            self.dataloader.load_state_dict(torch.load(path)["dataloader"])
        return ok


def fragment_llm(model, num_fragments: int) -> list[list[torch.nn.Parameter]]:
    """Split a decoder's parameters into ``num_fragments`` groups of consecutive blocks (embedding with the first,
    norm + head with the last): the fragments of streaming DiLoCo (parity: torchft/diloco/utils.py:112-136)."""
    blocks = list(model.layers.values())
    n = max(1, min(num_fragments, len(blocks)))
    per = (len(blocks) + n - 1) // n
    frags: list[list] = []
    for i in range(n):
        ps = [p for b in blocks[i * per:(i + 1) * per] for p in b.parameters()]
        frags.append(ps)
    if model.tok_embeddings is not None:
        frags[0] = list(model.tok_embeddings.parameters()) + frags[0]
    tail = [m for m in (model.norm, model.lm_head) if m is not None]
    seen = {id(p) for f in frags for p in f}
    frags[-1] += [p for m in tail for p in m.parameters() if id(p) not in seen]
    return [f for f in frags if f]


class FaultTolerantTrainer(Trainer):
    @dataclass(kw_only=True, slots=True)
    class Config(Trainer.Config):
        """The trainer's config plus ``--fault_tolerance.*`` (parity: torchft/config/job_config.py:15-87)."""
        fault_tolerance: FaultToleranceConfig = field(default_factory=FaultToleranceConfig)

    def __init__(self, config: "Trainer.Config", *, fault_tolerance: FaultToleranceConfig | None = None, store=None, **kw):
        super().__init__(config, **kw)
        ft = fault_tolerance or getattr(config, "fault_tolerance", None) or FaultToleranceConfig()
        self.ft = ft
        self.manager = None
        self.semi_sync: list = []
        if not ft.enable:
            return
        if store is None:
            from torch.distributed import TCPStore

            # one store for all replica groups; every rank talks to it under its own key prefix
            store = TCPStore(ft.store_addr, ft.store_port, is_master=(ft.replica_id == 0 and self.pdims.rank == 0),
                             timeout=timedelta(seconds=ft.quorum_timeout_s + 30), wait_for_workers=False)
        from torch.distributed import PrefixStore

        self.manager = FTManager(PrefixStore(f"rank{self.pdims.rank}", store), ft.replica_id, ft.group_size,
                                 heartbeat_timeout=ft.heartbeat_timeout_s, quorum_timeout=ft.quorum_timeout_s,
                                 min_replicas=ft.min_replica_size)
        self.manager.start_heartbeat_thread()
        self.optimizers = FTOptimizersContainer(self.optimizers, self.manager)
        self.checkpointer = FTCheckpointManager(self.checkpointer, self.dataloader, ft.replica_id, config.dump_folder)
        if ft.semi_sync_method:
            cls = {"local_sgd": LocalSGD, "diloco": DiLoCo}[ft.semi_sync_method]
            masters = [u.master for e in self.engines for u in e.units]       # the fp32 truth of every shard
            self.semi_sync = [cls(self.manager, masters, ft.sync_steps)]
        else:
            for e in self.engines:
                self._wrap_finalize(e)

    def _wrap_finalize(self, engine) -> None:
        """Average the reduced gradient shards over the live replicas right after the in-group reduction."""
        inner = engine.finalize_grads
        mgr = self.manager

        def finalize_grads():
            inner()
            grads = [engine._grad_of(u) for u in engine.units if u.grad_shard_valid]
            if grads and mgr.num_participants() > 1:
                mgr.allreduce(grads)

        engine.finalize_grads = finalize_grads

    def train_step(self, data_iterator) -> None:
        super().train_step(data_iterator)
        for s in self.semi_sync:
            if s.step():
                for e in self.engines:
                    e.publish_params()        # the averaged fp32 shards become the compute weights
