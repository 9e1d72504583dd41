"""Replica membership and fault-tolerant gradient averaging.

Every replica group (one model copy, possibly itself sharded over many GPUs) runs one
``FTManager`` on its first rank.  Managers share a key-value store (``torch.distributed.TCPStore``
or anything with ``set / get / add / check``):

* ``heartbeat()`` stamps ``hb/<id>`` with the wall clock; a replica whose stamp is older than
  ``heartbeat_timeout`` is considered gone (one that has not reported yet is waited for during the
  start-up grace period of ``quorum_timeout``).
* ``start_quorum(step)`` registers the replica for the step, then the lowest-numbered live replica
  (the leader of that step) waits for the others (until they register or their heartbeat expires),
  publishes the member list under ``quorum/<step>`` and everybody adopts it: all members agree on
  who takes part before any gradient is exchanged.
* ``allreduce(tensors)`` averages tensors over the quorum.  The default transport moves bytes
  through the store, which needs no process group that contains a dead rank; ``comm_factory`` can
  supply a collective over a process group created among the members only
  (``dist.new_group(ranks, use_local_synchronization=True)``) for NCCL-speed averaging.
* ``should_commit()`` is False when the step saw a transport error or lost a member half-way; the
  caller then skips the optimizer step (the gradients of an incomplete average are discarded).

A failure is always observed on the host, between kernels: nothing here waits on a device.
Reference behaviour: torchtitan/experiments/torchft/manager.py:91-126 (torchft ``Manager``).
"""

from __future__ import annotations

import io
import time
from dataclasses import dataclass

import torch

__all__ = ["FTManager", "QuorumResult"]


@dataclass
class QuorumResult:
    step: int
    members: list[int]
    changed: bool


class FTManager:
    def __init__(self, store, replica_id: int, num_replicas: int, *, heartbeat_timeout: float = 5.0,
                 quorum_timeout: float = 30.0, min_replicas: int = 1, comm_factory=None, clock=time.time):
        self.store = store
        self.id = replica_id
        self.n = num_replicas
        self.hb_timeout = heartbeat_timeout
        self.q_timeout = quorum_timeout
        self.min_replicas = min_replicas
        self.comm_factory = comm_factory
        self.clock = clock
        self.members: list[int] = list(range(num_replicas))
        self.step = -1
        self._errored = False
        self._comm = None
        self._t0 = clock()
        self._hb_thread = None
        self.heartbeat()

    # -- liveness ------------------------------------------------------------------------
    def heartbeat(self) -> None:
        self.store.set(f"hb/{self.id}", repr(self.clock()))

    def start_heartbeat_thread(self) -> None:
        """Beat from a daemon thread, so that a replica busy inside a long training step is not taken for dead.
        The thread ends with the process: a replica that exits (or is killed) stops beating."""
        import threading

        if self._hb_thread is not None:
            return

        def loop():
            while True:
                try:
                    self.heartbeat()
                except Exception:
                    return
                time.sleep(max(0.05, self.hb_timeout / 4))

        self._hb_thread = threading.Thread(target=loop, daemon=True)
        self._hb_thread.start()

    def _alive(self, rid: int) -> bool:
        if rid == self.id:
            return True
        key = f"hb/{rid}"
        if not self.store.check([key]):
            # a replica that has never reported is given the quorum timeout to come up
            return self.clock() - self._t0 < self.q_timeout
        return self.clock() - float(self.store.get(key).decode()) <= self.hb_timeout

    # -- quorum ---------------------------------------------------------------------------
    def start_quorum(self, step: int) -> QuorumResult:
        self.step = step
        self._errored = False
        self.heartbeat()
        self.store.set(f"join/{step}/{self.id}", "1")
        deadline = self.clock() + self.q_timeout
        qkey = f"quorum/{step}"
        while True:
            if self.store.check([qkey]):
                members = [int(x) for x in self.store.get(qkey).decode().split(",") if x]
                break
            live = [r for r in range(self.n) if self._alive(r)]
            if live and live[0] == self.id:
                # leader of this step: wait until every live replica has joined, or stopped beating
                joined = [r for r in live if self.store.check([f"join/{step}/{r}"])]
                if len(joined) == len(live) or self.clock() > deadline:
                    members = joined
                    self.store.set(qkey, ",".join(str(r) for r in members))
                    break
            if self.clock() > deadline + self.hb_timeout:
                raise TimeoutError(f"replica {self.id}: no quorum for step {step}")
            self.heartbeat()
            time.sleep(0.01)
        if self.id not in members:
            raise RuntimeError(f"replica {self.id} was left out of the quorum of step {step}; it must restart "
                               "from a live replica's checkpoint")
        if len(members) < self.min_replicas:
            raise RuntimeError(f"quorum of step {step} has {len(members)} replicas, fewer than min_replicas")
        changed = members != self.members
        self.members = members
        if changed and self.comm_factory is not None:
            self._comm = self.comm_factory(members)
        return QuorumResult(step, members, changed)

    # -- data ------------------------------------------------------------------------------
    def allreduce(self, tensors: list[torch.Tensor], tag: str = "g") -> None:
        """In-place average of ``tensors`` over the quorum of the current step."""
        if len(self.members) == 1:
            return
        try:
            if self._comm is not None:
                self._comm(tensors, len(self.members))
                return
            self._store_average(tensors, tag)
        except Exception:
            self._errored = True
            raise

    def _store_average(self, tensors, tag) -> None:
        buf = io.BytesIO()
        torch.save([t.detach().cpu() for t in tensors], buf)
        blob = buf.getvalue()
        # the store is a control-plane service: large payloads travel in 1 MiB parts, the part count last
        parts = [blob[i:i + (1 << 20)] for i in range(0, len(blob), 1 << 20)] or [b""]
        for i, part in enumerate(parts):
            self.store.set(f"ar/{self.step}/{tag}/{self.id}/{i}", part)
        self.store.set(f"ar/{self.step}/{tag}/{self.id}", str(len(parts)))
        acc = None
        deadline = self.clock() + self.q_timeout
        for r in self.members:
            key = f"ar/{self.step}/{tag}/{r}"
            while not self.store.check([key]):
                if not self._alive(r) or self.clock() > deadline:
                    self._errored = True
                    raise RuntimeError(f"replica {r} left during the average of step {self.step}")
                self.heartbeat()
                time.sleep(0.005)
            n_parts = int(self.store.get(key).decode())
            data = b"".join(self.store.get(f"{key}/{i}") for i in range(n_parts))
            vals = torch.load(io.BytesIO(data))
            acc = vals if acc is None else [a + v for a, v in zip(acc, vals)]
        for t, a in zip(tensors, acc):
            t.copy_((a / len(self.members)).to(t.dtype))

    def should_commit(self) -> bool:
        return not self._errored

    def num_participants(self) -> int:
        return len(self.members)
