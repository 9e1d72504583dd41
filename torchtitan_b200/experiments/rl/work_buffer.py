"""The buffer between the data-input loop, the rollout workers and the batcher of the asynchronous controller.

Every prompt group is an entry that moves ``waiting -> inflight -> finalized`` and is then taken by the batcher.
Independently of that, every admitted group holds one of ``max_active_rollout_groups`` *active slots* from
``add_work`` until ``release_active_groups`` (called after the generators pulled the weights trained on it, or at
once when the group turned out untrainable).  Holding the slot through training is what bounds staleness: no more
than the budget can be anywhere in the pipeline (buffer, batch queue, trainer), so no sample is generated that is
already too old when it is trained on.

The batcher takes the oldest finalized group whose id lies in ``[head, head + window_size - 1]`` where ``head``
is the oldest entry still in the buffer: ``window_size = 1`` is strict FIFO, a larger window lets finished groups
overtake a slow head without letting the head starve (the window does not slide past it).

Parity: torchtitan/experiments/rl/components/work_buffer.py:23-276.
"""

from __future__ import annotations

import asyncio
from collections import OrderedDict
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

from torchtitan_b200.config import Configurable

from . import metrics as m
from .records import RolloutGroup

__all__ = ["RolloutGroupWork", "RolloutGroupWorkBuffer"]


class _State(Enum):
    WAITING = 0
    INFLIGHT = 1
    FINALIZED = 2


@dataclass(slots=True)
class RolloutGroupWork:
    group_id: int
    sample: Any                                   # the dataset sample, passed unchanged to the environments
    state: _State = field(default=_State.WAITING, init=False)
    rollout_group: RolloutGroup | None = field(default=None, init=False)


class RolloutGroupWorkBuffer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass                                      # capacity and window are derived by the controller

    def __init__(self, config: Config | None = None, *, max_active_rollout_groups: int, window_size: int = 1):
        if not 1 <= window_size <= max_active_rollout_groups:
            raise ValueError(f"window_size must lie in [1, {max_active_rollout_groups}], got {window_size}")
        self.config = config
        self._cap, self._window = max_active_rollout_groups, window_size
        self._active = self._peak = 0
        self._work: OrderedDict[int, RolloutGroupWork] = OrderedDict()
        self._cond = asyncio.Condition()
        self._closed = False
        self.released: dict[str, int] = {}

    async def wait_for_slot(self) -> bool:
        """True when one more group may be admitted, False once the buffer is closed."""
        async with self._cond:
            await self._cond.wait_for(lambda: self._closed or self._active < self._cap)
            return not self._closed

    async def add_work(self, work: RolloutGroupWork) -> None:
        async with self._cond:
            if self._active >= self._cap:
                raise RuntimeError("add_work without a free active slot (call wait_for_slot first)")
            self._active += 1
            self._peak = max(self._peak, self._active)
            self._work[work.group_id] = work
            self._cond.notify_all()

    async def claim_next(self) -> RolloutGroupWork | None:
        """Oldest waiting group, marked inflight; None once closed."""
        async with self._cond:
            while True:
                if self._closed:
                    return None
                for w in self._work.values():
                    if w.state is _State.WAITING:
                        w.state = _State.INFLIGHT
                        return w
                await self._cond.wait()

    async def finalize_work(self, group: RolloutGroup) -> None:
        async with self._cond:
            w = self._work.get(group.group_id)
            if w is None:
                return
            w.rollout_group, w.state = group, _State.FINALIZED
            self._cond.notify_all()

    async def take_finalized(self) -> RolloutGroup | None:
        async with self._cond:
            while True:
                if self._closed:
                    return None
                if self._work:
                    end = next(iter(self._work)) + self._window - 1
                    for gid, w in self._work.items():
                        if gid > end:
                            break
                        if w.state is _State.FINALIZED:
                            del self._work[gid]
                            self._cond.notify_all()
                            return w.rollout_group
                await self._cond.wait()

    async def release_active_groups(self, count: int, *, reason: str) -> None:
        if count < 0:
            raise ValueError(f"count must be non-negative, got {count}")
        if count == 0:
            return
        async with self._cond:
            if count > self._active:
                raise RuntimeError(f"release_active_groups({count}) exceeds the {self._active} active groups")
            self._active -= count
            self.released[reason] = self.released.get(reason, 0) + count
            self._cond.notify_all()

    async def close(self) -> None:
        """Drops buffered work and wakes every waiter: ``wait_for_slot`` -> False, the others -> None."""
        async with self._cond:
            self._closed = True
            self._work.clear()
            self._cond.notify_all()

    def metrics(self) -> list[m.Metric]:
        states = [w.state for w in self._work.values()]
        out = [m.Metric("rollout_buffer/num_groups_waiting", m.NoReduce(states.count(_State.WAITING))),
               m.Metric("rollout_buffer/num_groups_inflight", m.NoReduce(states.count(_State.INFLIGHT))),
               m.Metric("rollout_buffer/num_groups_finalized", m.NoReduce(states.count(_State.FINALIZED))),
               m.Metric("rollout_buffer/active_slots_in_use_peak", m.NoReduce(self._peak)),
               m.Metric("rollout_buffer/available_active_slots", m.NoReduce(self._cap - self._active))]
        self._peak = self._active
        return out
