"""Request routing over generators, in two layers.

``InterGeneratorRouter`` spreads generation calls over generator replicas and fans the weight pull out to all of
them (``hot_swap``: pull while requests are in flight; otherwise each replica is taken out of rotation, drained of
its in-flight calls, updated and put back, the others keep serving).  ``IntraGeneratorRouter`` spreads the requests
of one replica over its data-parallel ranks and remembers which rank holds which request.

Strategies choose among candidates that expose ``reserved_load``: round robin; least loaded (ties go to the
candidate chosen longest ago, so that sessions started while everything is idle do not all land on the first
one); sticky sessions (a session key stays on its candidate while that candidate is routable: the prefix of a
multi-turn rollout is then already in that replica's cache; LRU-bounded map, fallback strategy for new keys).

Parity: torchtitan/experiments/rl/routing/strategies.py:36-193, intra_generator_router.py:22-93,
inter_generator_router.py:29-298 (there a Monarch actor in front of generator meshes; here an object of the
controller's event loop in front of engines of the same job).
"""

from __future__ import annotations

import abc
import asyncio
import itertools
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Sequence

from torchtitan_b200.config import Configurable

__all__ = ["RoutingContext", "RoutingStrategy", "RoundRobinRoutingStrategy", "LeastLoadedRoutingStrategy",
           "StickySessionRoutingStrategy", "IntraGeneratorRouter", "InterGeneratorRouter"]


@dataclass(frozen=True, kw_only=True, slots=True)
class RoutingContext:
    estimated_cost: int = 1
    session_id: str | None = None


class RoutingStrategy(Configurable, abc.ABC):
    @abc.abstractmethod
    def choose(self, ctx: RoutingContext, candidates: Sequence[Any]) -> Any:
        """One of the (non-empty) candidates; each has an integer ``reserved_load``."""


class RoundRobinRoutingStrategy(RoutingStrategy):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    def __init__(self, config=None, **_):
        self._n = itertools.count()

    def choose(self, ctx, candidates):
        return candidates[next(self._n) % len(candidates)]


class LeastLoadedRoutingStrategy(RoutingStrategy):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    def __init__(self, config=None, **_):
        self._tick = itertools.count()
        self._last: dict[int, int] = {}      # id(candidate) -> tick of its last selection

    def choose(self, ctx, candidates):
        low = min(c.reserved_load for c in candidates)
        # recency per candidate, not a position in the list: replicas leave and rejoin the list around weight pulls
        best = min((c for c in candidates if c.reserved_load == low), key=lambda c: self._last.get(id(c), -1))
        self._last[id(best)] = next(self._tick)
        return best


class StickySessionRoutingStrategy(RoutingStrategy):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        max_sessions: int = 4096
        fallback_strategy: Configurable.Config = field(default_factory=LeastLoadedRoutingStrategy.Config)

        def __post_init__(self):
            if self.max_sessions <= 0:
                raise ValueError(f"max_sessions must be positive, got {self.max_sessions}")

    def __init__(self, config: Config | None = None, **_):
        config = config or StickySessionRoutingStrategy.Config()
        self._max = config.max_sessions
        self._fallback = config.fallback_strategy.build()
        self._sessions: OrderedDict[str, Any] = OrderedDict()

    def choose(self, ctx, candidates):
        key = ctx.session_id
        if key is None:
            return self._fallback.choose(ctx, candidates)
        pinned = self._sessions.get(key)
        if pinned is not None and any(c is pinned for c in candidates):
            self._sessions.move_to_end(key)
            return pinned
        chosen = self._fallback.choose(ctx, candidates)      # new session, or its replica is out of rotation: re-pin
        self._sessions[key] = chosen
        self._sessions.move_to_end(key)
        if len(self._sessions) > self._max:
            self._sessions.popitem(last=False)
        return chosen


@dataclass(slots=True)
class _Rank:
    dp_rank: int
    reserved_load: int = 0


class IntraGeneratorRouter(Configurable):
    """``reserve(request_id)`` -> data-parallel rank (one unit of load on it), ``release(request_id)`` frees it.
    Not thread-safe: drive it from one event loop."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        strategy: Configurable.Config = field(default_factory=StickySessionRoutingStrategy.Config)

    def __init__(self, config: Config | None = None, *, dp_degree: int):
        if dp_degree <= 1:
            raise ValueError(f"dp_degree must be > 1, got {dp_degree}")
        self._strategy = (config or IntraGeneratorRouter.Config()).strategy.build()
        self._ranks = [_Rank(r) for r in range(dp_degree)]
        self._held: dict[str, int] = {}

    def reserve(self, request_id: str, *, routing_session_id: str | None = None) -> int:
        if request_id in self._held:
            raise ValueError(f"request {request_id!r} already holds a reservation")
        rank = self._strategy.choose(RoutingContext(session_id=routing_session_id), self._ranks)
        rank.reserved_load += 1
        self._held[request_id] = rank.dp_rank
        return rank.dp_rank

    def release(self, request_id: str) -> None:
        rank = self._ranks[self._held.pop(request_id)]
        rank.reserved_load -= 1
        assert rank.reserved_load >= 0, f"dp rank {rank.dp_rank}: negative load"

    def loads(self) -> list[int]:
        return [r.reserved_load for r in self._ranks]


@dataclass(eq=False, slots=True)
class _Replica:
    generator: Any
    reserved_load: int = 0
    serving: bool = True
    idle: asyncio.Event = field(default_factory=asyncio.Event)


class InterGeneratorRouter(Configurable):
    """``generators``: objects with ``async generate(prompt_token_ids, *, request_id, routing_session_id,
    sampling_config)`` and ``async pull_model_state_dict(policy_version)``."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        strategy: Configurable.Config = field(default_factory=LeastLoadedRoutingStrategy.Config)
        hot_swap: bool = True
        """Pull weights while generation is in flight.  Off: a replica finishes its routed calls before its pull;
        only single calls are waited for, so a multi-turn rollout can still see two policy versions."""

    def __init__(self, config: Config | None = None, *, generators: Sequence[Any]):
        self.config = config or InterGeneratorRouter.Config()
        if not generators:
            raise ValueError("InterGeneratorRouter needs at least one generator")
        self._replicas = [_Replica(g) for g in generators]
        for r in self._replicas:
            r.idle.set()
        self._strategy = self.config.strategy.build()
        self._any_serving = asyncio.Event()
        self._any_serving.set()

    def _candidates(self) -> list[_Replica]:
        return [r for r in self._replicas if r.serving]

    def _set_serving(self, r: _Replica, on: bool) -> None:
        r.serving = on
        if self._candidates():
            self._any_serving.set()
        else:
            self._any_serving.clear()

    def loads(self) -> list[int]:
        return [r.reserved_load for r in self._replicas]

    async def generate(self, prompt_token_ids: list[int], *, request_id: str, routing_session_id: str | None = None,
                       sampling_config=None, estimated_cost: int = 1):
        if estimated_cost < 0:
            raise ValueError(f"estimated_cost must be non-negative, got {estimated_cost}")
        await self._any_serving.wait()
        r = self._strategy.choose(RoutingContext(estimated_cost=estimated_cost, session_id=routing_session_id),
                                  self._candidates())
        if r.reserved_load == 0:
            r.idle.clear()
        r.reserved_load += estimated_cost
        try:
            return await r.generator.generate(prompt_token_ids, request_id=request_id,
                                              routing_session_id=routing_session_id, sampling_config=sampling_config)
        finally:                                  # a failed call must not leave load behind
            r.reserved_load -= estimated_cost
            if r.reserved_load == 0:
                r.idle.set()

    async def pull_model_state_dict(self, policy_version: int) -> None:
        async def one(r: _Replica):
            if self.config.hot_swap:
                await r.generator.pull_model_state_dict(policy_version)
                return
            self._set_serving(r, False)
            try:
                await r.idle.wait()
                await r.generator.pull_model_state_dict(policy_version)
            finally:
                self._set_serving(r, True)

        await asyncio.gather(*(one(r) for r in self._replicas))

    async def fanout(self, method: str, *args, return_exceptions: bool = False, **kw) -> list:
        return await asyncio.gather(*(getattr(r.generator, method)(*args, **kw) for r in self._replicas),
                                    return_exceptions=return_exceptions)

    async def close_generators(self) -> list:
        return await self.fanout("close", return_exceptions=True)
