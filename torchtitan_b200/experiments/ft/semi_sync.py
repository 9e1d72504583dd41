"""Semi-synchronous training over fault-tolerant replicas.

``LocalSGD``: replicas train independently and average their parameters every ``sync_every`` steps.
``DiLoCo``: every ``sync_every`` inner steps the pseudo-gradient ``global - local`` is averaged over
the live replicas and an outer optimizer (SGD with Nesterov momentum by default) updates the
global parameters, which the replicas then adopt.  Parity: torchft ``LocalSGD`` / ``DiLoCo`` as
wired by torchtitan/experiments/torchft."""

from __future__ import annotations

import torch

from .manager import FTManager

__all__ = ["LocalSGD", "DiLoCo"]


class LocalSGD:
    def __init__(self, manager: FTManager, params, sync_every: int):
        self.m = manager
        self.params = [p for p in params]
        self.sync_every = sync_every
        self.local_step = 0

    def step(self) -> bool:
        """Call after every inner optimizer step; returns True when a synchronisation happened."""
        self.local_step += 1
        if self.local_step % self.sync_every:
            return False
        self.m.start_quorum(self.local_step // self.sync_every)
        self._sync()
        return True

    def _sync(self) -> None:
        with torch.no_grad():
            self.m.allreduce([p.data for p in self.params], tag="p")


class DiLoCo(LocalSGD):
    def __init__(self, manager: FTManager, params, sync_every: int, outer_lr: float = 0.7, momentum: float = 0.9):
        super().__init__(manager, params, sync_every)
        self.global_params = [p.detach().clone() for p in self.params]
        for g in self.global_params:
            g.requires_grad_(True)
        self.outer = torch.optim.SGD(self.global_params, lr=outer_lr, momentum=momentum, nesterov=momentum > 0)

    def _sync(self) -> None:
        with torch.no_grad():
            pseudo = [g.detach() - p.detach() for g, p in zip(self.global_params, self.params)]
        self.m.allreduce(pseudo, tag="d")
        if not self.m.should_commit():
            return
        for g, d in zip(self.global_params, pseudo):
            g.grad = d
        self.outer.step()
        with torch.no_grad():
            for p, g in zip(self.params, self.global_params):
                p.copy_(g)
