"""A continuous-batching generation engine on the training model's own modules.

Requests arrive through ``await engine.generate(prompt_token_ids, ...)`` at any time.  Every engine step admits
waiting requests (up to ``max_num_seqs`` sequences and ``max_batched_tokens`` prompt rows), concatenates the new
prompts and one row for each sequence already decoding into ONE flat token stream, and runs the decoder once over
it: projections, feed-forward / expert layers and the output projection see all rows together (weights are read
once per step for all sequences), the attention core runs per sequence against that sequence's key/value cache
(``models.common.attention.BatchedKVCache``).  Only the last row of each sequence reaches the output projection.
Sampling (temperature, top-k, top-p, per-request seed) happens per sequence; a sequence ends on EOS, a stop token,
a stop sequence (``finish_reason = "stop"``), its token limit (``"length"``) or engine shutdown (``"abort"``).

New weights are applied between two steps (``pull_model_state_dict``): sequences in flight keep their caches and
continue under the new policy, and each completion reports the oldest and newest policy version its tokens were
sampled under.

Parity: torchtitan/experiments/rl/actors/generator.py:174-1460 (vLLM engine loop, request dispatcher, sampling
config, weight pull; the reference runs vLLM with the trainer's model definitions registered into it, here the
engine *is* the trainer's model code).
"""

from __future__ import annotations

import asyncio
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from . import metrics as m
from .generator import frozen_router_counters
from .records import Completion

__all__ = ["SamplingConfig", "GenerationEngine", "DataParallelEngine", "place_model_"]


def place_model_(model, device, param_dtype: torch.dtype | None = None):
    """Move ``model`` to ``device`` and cast its floating-point *parameters* to ``param_dtype``.  Buffers keep their
    dtype: the rotary tables (and the routers' selection bias) are fp32 by contract of the kernels that read them,
    which ``model.to(dtype=...)`` would silently break."""
    model.to(device)
    if param_dtype is not None:
        for p in model.parameters():
            if p.is_floating_point() and p.dtype != param_dtype:
                p.data = p.data.to(param_dtype)
    return model


@dataclass(kw_only=True, slots=True)
class SamplingConfig:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    max_tokens: int = 128
    seed: int | None = None
    stop_token_ids: list[int] = field(default_factory=list)
    stop_sequences: list[list[int]] = field(default_factory=list)


@dataclass(eq=False, slots=True)
class _Seq:
    request_id: str
    pending: list[int]                      # rows to feed at the next step (whole prompt, then the last token)
    sampling: SamplingConfig
    future: Any
    loop: Any
    cache: Any
    pos: int = 0
    out_ids: list[int] = field(default_factory=list)
    out_lps: list[float] = field(default_factory=list)
    rng: torch.Generator | None = None
    v_min: int | None = None
    v_max: int | None = None
    t_arrive: float = 0.0
    t_first: float | None = None


def sample_token(logits: torch.Tensor, s: SamplingConfig, rng: torch.Generator | None) -> tuple[int, float]:
    """One token from ``logits[V]`` (fp32).  The reported log-probability is that of the token under the
    distribution actually sampled from (after temperature and truncation), which is what the importance ratio of
    the policy loss needs."""
    if s.temperature <= 0:
        lp = torch.log_softmax(logits, -1)
        t = int(lp.argmax())
        return t, float(lp[t])
    logits = logits / s.temperature
    if s.top_k and s.top_k < logits.numel():
        kth = logits.topk(s.top_k).values[-1]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if s.top_p < 1.0:
        srt, idx = logits.sort(descending=True)
        cum = torch.softmax(srt, -1).cumsum(-1)
        drop = cum - torch.softmax(srt, -1) >= s.top_p          # keep the first token that crosses top_p
        logits = logits.masked_fill(torch.zeros_like(drop).scatter(0, idx, drop), float("-inf"))
    probs = torch.softmax(logits, -1)
    t = int(torch.multinomial(probs.cpu(), 1, generator=rng)[0])
    return t, float(torch.log(probs[t]))


class GenerationEngine(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        max_num_seqs: int = 64
        max_batched_tokens: int = 8192
        """Prompt rows admitted per step (a single longer prompt is still admitted alone)."""
        threaded: bool = True
        """Run engine steps in a worker thread so that the controller's event loop (and a trainer on another
        device or stream) keeps going.  Must be off when the engine shares its model object with the trainer."""
        sampling: SamplingConfig = field(default_factory=SamplingConfig)

    def __init__(self, config: Config | None = None, *, model, eos_id: int | None = None,
                 weight_source: Callable[["GenerationEngine"], None] | None = None):
        self.config = config or GenerationEngine.Config()
        self.model, self.eos_id, self.weight_source = model, eos_id, weight_source
        # positions beyond the rotary tables are an error in the kernels: sequences stop there ("length")
        self.max_context = getattr(getattr(model, "config", None), "max_context_length", None)
        self.policy_version = 0
        self._waiting: list[_Seq] = []
        self._running: list[_Seq] = []
        self._lock = threading.Lock()            # guards _waiting / _pending_pull between the loop thread and callers
        self._pending_pull: list[tuple[int, Any, Any]] = []
        self._wake: asyncio.Event | None = None
        self._task: asyncio.Task | None = None
        self._closed = False
        self.steps = 0
        self.tokens_generated = 0

    # -- public API ----------------------------------------------------------------------------------------------
    async def generate(self, prompt_token_ids: list[int], *, request_id: str, routing_session_id: str | None = None,
                       sampling_config: SamplingConfig | None = None) -> Completion:
        from torchtitan_b200.models.common.attention import KVCache

        if self._closed:
            return Completion(request_id=request_id, token_ids=[], token_logprobs=[], finish_reason="abort",
                              min_policy_version=self.policy_version, max_policy_version=self.policy_version)
        if not prompt_token_ids:
            raise ValueError(f"{request_id}: empty prompt")
        if self.max_context and len(prompt_token_ids) >= self.max_context:
            raise ValueError(f"{request_id}: the prompt has {len(prompt_token_ids)} tokens, the model's context is "
                             f"{self.max_context}")
        s = sampling_config or self.config.sampling
        loop = asyncio.get_running_loop()
        seq = _Seq(request_id=request_id, pending=list(prompt_token_ids), sampling=s, future=loop.create_future(),
                   loop=loop, cache=KVCache(), t_arrive=time.perf_counter(),
                   rng=None if s.seed is None else torch.Generator().manual_seed(s.seed))
        with self._lock:
            self._waiting.append(seq)
        self._ensure_loop()
        self._wake.set()
        return await seq.future

    async def pull_model_state_dict(self, policy_version: int) -> None:
        """Applied at the next step boundary (at once when the engine is idle)."""
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self._pending_pull.append((policy_version, fut, loop))
        self._ensure_loop()
        self._wake.set()
        await fut

    async def close(self) -> None:
        self._closed = True
        if self._wake is not None:
            self._wake.set()
        if self._task is not None:
            await asyncio.gather(self._task, return_exceptions=True)
        with self._lock:
            left, self._waiting, self._running = self._waiting + self._running, [], []
        for seq in left:
            self._finish(seq, "abort")

    # -- loop ----------------------------------------------------------------------------------------------------
    def _ensure_loop(self) -> None:
        if self._wake is None:
            self._wake = asyncio.Event()
        if self._task is None or self._task.done():
            self._task = asyncio.get_running_loop().create_task(self._run(), name="generation_engine")

    async def _run(self) -> None:
        while not self._closed:
            with self._lock:
                busy = bool(self._waiting or self._running or self._pending_pull)
            if not busy:
                self._wake.clear()
                with self._lock:                 # a request may have arrived between the check and the clear
                    busy = bool(self._waiting or self._running or self._pending_pull)
                if not busy:
                    await self._wake.wait()
                    continue
            try:
                if self.config.threaded:
                    await asyncio.to_thread(self.step)
                else:
                    self.step()
                    await asyncio.sleep(0)
            except Exception as e:
                # a failed forward leaves the caches of the sequences in flight in an unknown state: their requests
                # fail with the error (instead of waiting forever), the engine stays up for new ones
                logger.exception("generation engine step failed")
                self._fail_inflight(e)

    def _fail_inflight(self, error: Exception) -> None:
        with self._lock:
            hit, self._running = self._running, []
        for seq in hit:
            seq.cache = None
            if not seq.future.done():
                seq.future.set_exception(RuntimeError(f"{seq.request_id}: generation failed: {error!r}"))

    def _apply_pulls(self) -> None:
        with self._lock:
            pulls, self._pending_pull = self._pending_pull, []
        for version, fut, loop in pulls:
            try:
                if self.weight_source is not None:
                    self.weight_source(self)
                self.policy_version = version
                loop.call_soon_threadsafe(lambda f=fut: f.done() or f.set_result(None))
            except Exception as e:              # the caller of the pull sees the failure
                loop.call_soon_threadsafe(lambda f=fut, e=e: f.done() or f.set_exception(e))

    @torch.no_grad()
    def step(self) -> int:
        """One engine iteration; returns the number of sequences that produced a token."""
        from torchtitan_b200.models.common.attention import AttentionContext, BatchedKVCache

        self._apply_pulls()
        c = self.config
        with self._lock:
            budget = c.max_batched_tokens
            while self._waiting and len(self._running) < c.max_num_seqs:
                n = len(self._waiting[0].pending)
                if n > budget and budget < c.max_batched_tokens:
                    break                          # next step; a prompt longer than the whole budget goes alone
                budget -= n
                self._running.append(self._waiting.pop(0))
        seqs = self._running
        if not seqs:
            return 0
        dev = next(self.model.parameters()).device
        rows = [len(s.pending) for s in seqs]
        tokens = torch.tensor([t for s in seqs for t in s.pending], dtype=torch.long, device=dev)
        positions = torch.cat([torch.arange(s.pos, s.pos + n) for s, n in zip(seqs, rows)]).to(dev)
        last = torch.tensor(rows, device=dev).cumsum(0) - 1
        was_training = self.model.training
        self.model.eval()
        ctx = AttentionContext(kv_cache=BatchedKVCache([s.cache for s in seqs], rows))
        try:
            with frozen_router_counters(self.model):
                if hasattr(self.model, "output_logits") and getattr(self.model, "tp", None) is None:
                    logits = self.model.output_logits(self.model(tokens, positions, ctx, return_hidden=True)[last])
                else:
                    logits = self.model(tokens, positions, ctx)[last]
        finally:
            self.model.train(was_training)
        logits = logits.float()
        now = time.perf_counter()
        still = []
        for i, s in enumerate(seqs):
            tok, lp = sample_token(logits[i], s.sampling, s.rng)
            s.pos += rows[i]
            s.out_ids.append(tok)
            s.out_lps.append(lp)
            s.pending = [tok]
            s.t_first = s.t_first or now
            v = self.policy_version
            s.v_min = v if s.v_min is None else min(s.v_min, v)
            s.v_max = v if s.v_max is None else max(s.v_max, v)
            reason = self._finish_reason(s, tok)
            if reason:
                self._finish(s, reason)
            else:
                still.append(s)
        with self._lock:
            self._running = still
        self.steps += 1
        self.tokens_generated += len(seqs)
        return len(seqs)

    def _finish_reason(self, s: _Seq, tok: int) -> str | None:
        sc = s.sampling
        if (self.eos_id is not None and tok == self.eos_id) or tok in sc.stop_token_ids:
            return "stop"
        for stop in sc.stop_sequences:
            if stop and s.out_ids[-len(stop):] == stop:
                return "stop"
        if self.max_context and s.pos + 1 >= self.max_context:      # the next row would be past the context
            return "length"
        return "length" if len(s.out_ids) >= sc.max_tokens else None

    def _finish(self, s: _Seq, reason: str) -> None:
        now = time.perf_counter()
        v0 = self.policy_version if s.v_min is None else s.v_min
        v1 = self.policy_version if s.v_max is None else s.v_max
        done = Completion(request_id=s.request_id, token_ids=s.out_ids, token_logprobs=s.out_lps, finish_reason=reason,
                          min_policy_version=v0, max_policy_version=v1, metrics=[
                              m.Metric("generator/time_to_first_token_s", m.Mean((s.t_first or now) - s.t_arrive)),
                              m.Metric("generator/request_latency_s", m.Mean(now - s.t_arrive)),
                              m.Metric("generator/response_length", m.Mean(len(s.out_ids))),
                              m.Metric("generator/response_length", m.Max(len(s.out_ids)))])
        s.cache = None
        try:
            s.loop.call_soon_threadsafe(lambda: s.future.done() or s.future.set_result(done))
        except RuntimeError:                        # the request's event loop is gone
            logger.warning(f"{s.request_id}: completion dropped, its event loop is closed")


class DataParallelEngine:
    """One generator made of several engines holding the same weights (one per GPU): layer two of the routing
    design.  Each request is placed on a data-parallel rank by an ``IntraGeneratorRouter`` (sticky sessions by
    default, so the turns of one rollout reuse one rank) and released when it completes; weight pulls and ``close``
    fan out to every rank.  It has the interface of a single engine, so an ``InterGeneratorRouter`` can sit in front
    of several of them."""

    def __init__(self, engines: list[GenerationEngine], router_config=None):
        from .routing import IntraGeneratorRouter

        if len(engines) < 2:
            raise ValueError("DataParallelEngine needs at least two engines (use the engine itself otherwise)")
        self.engines = list(engines)
        self.router = IntraGeneratorRouter(router_config, dp_degree=len(engines))

    @property
    def policy_version(self) -> int:
        return min(e.policy_version for e in self.engines)

    async def generate(self, prompt_token_ids: list[int], *, request_id: str, routing_session_id: str | None = None,
                       sampling_config: SamplingConfig | None = None) -> Completion:
        rank = self.router.reserve(request_id, routing_session_id=routing_session_id)
        try:
            return await self.engines[rank].generate(prompt_token_ids, request_id=request_id,
                                                     routing_session_id=routing_session_id, sampling_config=sampling_config)
        finally:
            self.router.release(request_id)

    async def pull_model_state_dict(self, policy_version: int) -> None:
        await asyncio.gather(*(e.pull_model_state_dict(policy_version) for e in self.engines))

    async def close(self) -> None:
        await asyncio.gather(*(e.close() for e in self.engines))
