"""Sharded data parallelism with flat per-unit buffers (ZeRO-style, B200 layout).

Design.  Parameters are grouped into *units* (embedding, each transformer block,
final norm + lm_head -- the same unit structure the reference gives FSDP2,
torchtitan/distributed/fsdp.py:168-381).  Per unit there are

* ``flat_param``  full-size buffer in the compute dtype (bf16); module parameters
  are views into it.  Two layouts, chosen by ``parallelism.fsdp_reshard_after_forward``
  (reference: torchtitan/distributed/fsdp.py:112-166):

  - *resident* (``never``; also ``default`` while the replicated bf16 weights and
    gradients take less than a third of the device memory): every unit keeps its own
    full-size ``flat_param`` and ``flat_grad``.  With 180 GB of HBM the weights of the
    8B - 70B models stay resident, so there is no all-gather on the forward critical
    path: the gathered weights are refreshed once per optimizer step.
  - *sharded* (``always``, and ``default`` for models that do not fit): a rank keeps
    only its 1/N ``param_shard`` of every unit between uses (ZeRO-3 / FSDP2).  The
    full-size buffers come from two rotating slots per sharding group, sized for the
    largest unit; unit k+1 is gathered into the other slot on the communication stream
    while unit k computes (forward order in forward, reverse order in backward), and
    gradients are reduce-scattered out of two rotating gradient slots.  Parameter
    shards change only in the optimizer, so the gathers need no cross-rank barrier
    besides the one that ends the optimizer step.
* ``flat_grad``   full-size local gradient buffer (compute dtype).  The linear
  backward writes weight gradients straight into it (``main_grad`` views).
* ``master`` / ``exp_avg`` / ``exp_avg_sq`` / ``grad_shard``: this rank's 1/N slice
  in fp32 (optimizer moments optionally bf16).

Sharding is by *flat offset*: rank r owns elements ``[r*S, (r+1)*S)`` of the padded
flat buffer, so both collectives run in place on the buffers without copy-in /
copy-out, and the same layout is what the in-kernel NVLink path reads and writes.

Per optimizer step and unit:  local grads --(reduce-scatter, fp32 accumulate)-->
``grad_shard``; global grad-norm from per-unit partial sums; AdamW on the shard
which also writes the updated bf16 weights into ``flat_param``; all-gather of
``flat_param``.  Gradient division is never applied: the loss is already divided
by the global token count (torchtitan/distributed/fsdp.py:85-99).

Two communication back ends: ``nccl`` (library collectives; also ``gloo`` on CPU)
and ``nvlink`` (peer loads / stores from our own kernels over symmetric memory,
:mod:`torchtitan_b200.parallel.symm`).
"""

from __future__ import annotations

import contextlib
import math
import re
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

import torch
import torch.distributed as dist
import torch.nn as nn

from torchtitan_b200.models.common.module import InitSpec, iter_checkpoint_slices, materialize_param
from torchtitan_b200.ops import optim as optim_ops

__all__ = ["ShardedModel", "FlatUnit", "ParamSlot", "UnitSpec"]

_ALIGN = 128  # elements; keeps every shard boundary 256-byte aligned for bf16


@dataclass
class ParamSlot:
    fqn: str
    param: nn.Parameter
    shape: tuple[int, ...]
    numel: int
    offset: int  # element offset inside the unit's flat buffer
    init: InitSpec
    tp_slices: Any = None  # (dim, [(a,b),...], global_shape) when tensor-parallel sharded
    tp_replicated: bool = False
    group_idx: int = 0  # optimizer param group


@dataclass
class UnitSpec:
    name: str
    modules: list[nn.Module]
    group_name: str = "fsdp"  # which mesh axis shards this unit ("fsdp" or "efsdp")
    param_filter: Callable[[str, nn.Parameter], bool] | None = None


class FlatUnit:
    def __init__(self, name: str, slots: list[ParamSlot], group, group_size: int, group_rank: int,
                 replicate_group=None):
        self.name = name
        self.slots = slots
        self.group = group
        self.size = group_size
        self.rank = group_rank
        self.replicate_group = replicate_group
        total = sum(s.numel for s in slots)
        quantum = _ALIGN * group_size
        self.numel = total
        self.padded = max(quantum, (total + quantum - 1) // quantum * quantum)
        self.shard_numel = self.padded // group_size
        self.flat_param: torch.Tensor | None = None
        self.flat_grad: torch.Tensor | None = None
        self.master: torch.Tensor | None = None
        self.grad_shard: torch.Tensor | None = None
        self.exp_avg: torch.Tensor | None = None
        self.exp_avg_sq: torch.Tensor | None = None
        self.rep_numel = 0  # leading elements that are replicated across tensor-parallel ranks
        self.rep_reduce_numel = 0  # the part of them whose gradients are per-rank parts to be summed over tp
        self.pending = False  # gradients written, reduction not yet launched
        self.grad_shard_valid = False
        self.sumsq: torch.Tensor | None = None  # [2]: (tp-replicated part, rest)
        # sharded-parameter layout only
        self.param_shard: torch.Tensor | None = None   # this rank's 1/N of the parameters, compute dtype
        self.pool: "_SlotPool | None" = None
        self.slot = 0
        self.gather_dst: torch.Tensor | None = None    # alias of flat_param with its own version counter
        self.private_grad = False                      # gradients in an own buffer instead of a rotating slot
        self.ready = None                              # event of the optimizer step still refreshing this unit
        self.hooked = False                            # a forward pre-hook of this unit exists

    # shard geometry -----------------------------------------------------
    @property
    def shard_start(self) -> int:
        return self.rank * self.shard_numel

    def shard_view(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.shard_start:self.shard_start + self.shard_numel]

    def slot_pieces(self, rank: int | None = None):
        """Intersections of this rank's shard with each parameter:
        ``(slot, param_flat_start, shard_start, length)``."""
        r = self.rank if rank is None else rank
        lo, hi = r * self.shard_numel, (r + 1) * self.shard_numel
        for s in self.slots:
            a, b = max(lo, s.offset), min(hi, s.offset + s.numel)
            if a < b:
                yield s, a - s.offset, a - lo, b - a


class ShardedModel:
    """Owns the flat buffers of a model (or pipeline stage) and its sharded optimizer state."""

    def __init__(self, model: nn.Module, units: list[UnitSpec], *, pdims, device: torch.device,
                 param_dtype: torch.dtype = torch.bfloat16, master_dtype: torch.dtype = torch.float32,
                 state_dtype: torch.dtype = torch.float32, seed: int = 0, comm: str = "nccl",
                 grad_accum_steps: int = 1, fqn_prefix: str = "", tp=None, offload_optimizer: bool = False,
                 reshard_after_forward: str = "never"):
        self.model = model
        if reshard_after_forward not in ("default", "always", "never"):
            raise ValueError("fsdp_reshard_after_forward must be 'default', 'always' or 'never'")
        self.reshard_policy = reshard_after_forward
        self.sharded_params = False     # decided in materialize()
        self._pools: dict[int, _SlotPool] = {}
        self._order: list[FlatUnit] = []   # units with sharded parameters, in execution order
        self._in_backward = False
        self._optimizer_inflight = False
        self._rs_unfenced = False     # reduce-scatters launched without their own trailing barrier in this pass
        # optimizer state (fp32 master weights and both moments) lives in pinned host memory and is
        # streamed through the GPU one unit at a time during the optimizer step
        self.offload_optimizer = bool(offload_optimizer) and device.type == "cuda"
        self.pdims = pdims
        self.device = device
        self.param_dtype = param_dtype
        self.state_dtype = state_dtype
        self.seed = seed
        self.comm = comm
        self.tp = tp
        self.grad_accum_steps = grad_accum_steps
        self.fqn_prefix = fqn_prefix
        self.units: list[FlatUnit] = []
        self.frozen: dict[str, nn.Parameter] = {}
        self.step_count = 0
        self._comm_stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self._fp32_tmp: list[torch.Tensor] = []
        self._tmp_idx = 0
        self._symm = None
        self._callback_queued = False
        self.defer_reduce = False
        self._build_units(units)

    # ------------------------------------------------------------------
    # construction
    # ------------------------------------------------------------------
    def _build_units(self, specs: list[UnitSpec]) -> None:
        fqn_of: dict[int, str] = {}
        for name, p in self.model.named_parameters(remove_duplicate=True):
            fqn_of[id(p)] = name
        claimed: set[int] = set()
        for spec in specs:
            slots: list[ParamSlot] = []
            plist: list[tuple[str, nn.Parameter]] = []
            for m in spec.modules:
                for _, p in m.named_parameters(remove_duplicate=True):
                    if id(p) in claimed or id(p) not in fqn_of:
                        continue
                    if spec.param_filter is not None and not spec.param_filter(fqn_of[id(p)], p):
                        continue
                    claimed.add(id(p))
                    plist.append((fqn_of[id(p)], p))
            trainable = [(n, p) for n, p in plist if p.requires_grad]
            for n, p in plist:
                if not p.requires_grad:
                    self.frozen[n] = p
            if not trainable:
                continue
            # tensor-parallel-replicated parameters first: the ones whose gradient is a per-rank part (summed with
            # one all-reduce over the leading range of the flat buffer), then the ones whose gradient is already
            # complete on every rank (no reduction; both kinds are counted once in the gradient norm)
            sp = self.tp is None or self.tp.sequence_parallel

            def _tp_class(p) -> int:
                if not getattr(p, "_replicated_over_tp", False):
                    return 2
                return 1 if (not sp and getattr(p, "_tp_grad_complete_without_sp", False)) else 0

            trainable.sort(key=lambda np_: _tp_class(np_[1]))
            off = 0
            rep = 0
            rep_reduce = 0
            for n, p in trainable:
                slot = ParamSlot(
                    fqn=n, param=p, shape=tuple(p.shape), numel=p.numel(), offset=off,
                    init=getattr(p, "_init_spec", None) or InitSpec(),
                    tp_slices=getattr(p, "_tp_slices", None),
                    tp_replicated=bool(getattr(p, "_replicated_over_tp", False)),
                )
                slots.append(slot)
                off += (p.numel() + 7) // 8 * 8  # keep every parameter 16-byte aligned
                if slot.tp_replicated:
                    rep = off
                    if _tp_class(p) == 0:
                        rep_reduce = off
            # compact numel accounting: last slot's padding is part of unit padding
            gname = spec.group_name
            group = self.pdims.group(gname)
            gsize = self.pdims.size(gname)
            grank = self.pdims.local_rank(gname) if gsize > 1 else 0
            rgroup = self.pdims.group("dp_replicate")
            unit = FlatUnit(spec.name, slots, group, gsize, grank, rgroup)
            quantum = _ALIGN * gsize
            unit.numel = off
            unit.padded = max(quantum, (off + quantum - 1) // quantum * quantum)
            unit.shard_numel = unit.padded // gsize
            unit.rep_numel = rep if (self.tp is not None and self.tp.size > 1) else 0
            unit.rep_reduce_numel = rep_reduce if (self.tp is not None and self.tp.size > 1) else 0
            self.units.append(unit)
        missing = [n for i, n in fqn_of.items() if i not in claimed]
        if missing:
            raise ValueError(f"parameters not assigned to any sharding unit: {missing[:5]} ...")

    def _decide_layout(self, pd: torch.dtype) -> bool:
        """True when parameters are kept sharded between uses (see the module docstring)."""
        multi = [u for u in self.units if u.size > 1]
        if not multi or self.reshard_policy == "never":
            return False
        if self.reshard_policy == "always":
            return True
        if self.device.type != "cuda":
            return False
        es = torch.empty(0, dtype=pd).element_size()
        replicated = sum(2 * u.padded * es for u in multi)
        return replicated > torch.cuda.get_device_properties(self.device).total_memory // 3

    def materialize(self, init: bool = True) -> None:
        """Allocate buffers, point module parameters at them, initialise the fp32 master shards."""
        dev, pd = self.device, self.param_dtype
        self.sharded_params = self._decide_layout(pd)
        use_symm = self.comm in ("nvlink", "auto") and dev.type == "cuda" and any(u.size > 1 for u in self.units)
        if use_symm:
            use_symm = self._setup_symmetric(pd)
        if self.sharded_params:
            # two parameter slots and two gradient slots per sharding group, each as large as the group's largest unit
            biggest: dict[int, int] = {}
            for u in self.units:
                if u.size > 1:
                    biggest[id(u.group)] = max(biggest.get(id(u.group), 0), u.padded)
            seen: dict[int, int] = {}
            for u in self.units:
                if u.size == 1:
                    continue
                key = id(u.group)
                if key not in self._pools:
                    n = biggest[key]
                    if use_symm:
                        grads = [self._symm.alloc(n, pd, u.group, tag=f"grad_slot{i}") for i in range(2)]
                    else:
                        grads = [torch.zeros(n, dtype=pd, device=dev) for _ in range(2)]
                    for g in grads:
                        g.zero_()
                    self._pools[key] = _SlotPool([torch.zeros(n, dtype=pd, device=dev) for _ in range(2)], grads)
                u.pool = self._pools[key]
                u.slot = seen.get(key, 0) % 2
                seen[key] = seen.get(key, 0) + 1
                self._order.append(u)
        replaced: dict[int, nn.Parameter] = {}
        for u in self.units:
            if u.pool is not None:
                u.flat_param = _alias(u.pool.param[u.slot], u.padded)
                u.gather_dst = _alias(u.pool.param[u.slot], u.padded)
                if u is self._order[0]:
                    # The first unit in execution order (the embedding on a first stage) may have no input that
                    # carries a gradient, so the end of its backward is only known when the whole backward has
                    # finished; its gradients get a buffer of their own instead of a rotating slot.
                    if use_symm:
                        u.flat_grad = self._symm.alloc(u.padded, pd, u.group, tag=f"{u.name}.grad")
                        u.flat_grad.zero_()
                    else:
                        u.flat_grad = torch.zeros(u.padded, dtype=pd, device=dev)
                    u.private_grad = True
                else:
                    u.flat_grad = _alias(u.pool.grad[u.slot], u.padded)
                if use_symm:
                    u.param_shard = self._symm.alloc(u.shard_numel, pd, u.group, tag=f"{u.name}.param_shard")
                    u.param_shard.zero_()
                else:
                    u.param_shard = torch.zeros(u.shard_numel, dtype=pd, device=dev)
            elif use_symm and u.size > 1:
                u.flat_param = self._symm.alloc(u.padded, pd, u.group, tag=f"{u.name}.param")
                u.flat_grad = self._symm.alloc(u.padded, pd, u.group, tag=f"{u.name}.grad")
                u.flat_param.zero_()
                u.flat_grad.zero_()
            else:
                u.flat_param = torch.zeros(u.padded, dtype=pd, device=dev)
                u.flat_grad = torch.zeros(u.padded, dtype=pd, device=dev)
            if self.offload_optimizer:
                u.master = torch.zeros(u.shard_numel, dtype=torch.float32, pin_memory=True)
            else:
                u.master = torch.zeros(u.shard_numel, dtype=torch.float32, device=dev)
            u.sumsq = torch.zeros(2, dtype=torch.float32, device=dev)
            # A separate fp32 gradient shard is needed whenever gradients are summed across
            # ranks or across microbatches; a lone owner with one microbatch lets the
            # optimizer read the local gradient buffer directly.
            if u.size > 1 or self.grad_accum_steps > 1 or u.replicate_group is not None:
                u.grad_shard = torch.zeros(u.shard_numel, dtype=torch.float32, device=dev)
            for s in u.slots:
                new = nn.Parameter(u.flat_param[s.offset:s.offset + s.numel].view(s.shape), requires_grad=True)
                for attr in ("_init_spec", "_tp_slices", "_replicated_over_tp", "_is_expert"):
                    if hasattr(s.param, attr):
                        setattr(new, attr, getattr(s.param, attr))
                new.main_grad = u.flat_grad[s.offset:s.offset + s.numel].view(s.shape)
                new._main_grad_written = False
                new._unit = u
                replaced[id(s.param)] = new
                s.param = new
        for name, p in list(self.frozen.items()):
            spec = getattr(p, "_init_spec", None) or InitSpec()
            full = self._materialize_full(name, p, spec)
            new = nn.Parameter(full.to(pd), requires_grad=False)
            replaced[id(p)] = new
            self.frozen[name] = new
        _swap_parameters(self.model, replaced)
        if init:
            self.init_weights()

    def _setup_symmetric(self, pd: torch.dtype) -> bool:
        """Create the symmetric arenas; with ``comm="auto"`` fall back to NCCL when any rank fails."""
        from . import symm

        ok = True
        err: Exception | None = None
        try:
            if not symm.symm_available():
                raise RuntimeError("torch symmetric memory is unavailable")
            arena = symm.SymmetricArena(self.pdims, self.device)
            es = torch.empty(0, dtype=pd).element_size()
            groups = {}
            biggest: dict[int, int] = {}
            for u in self.units:
                if u.size > 1:
                    groups[id(u.group)] = u.group
                    if self.sharded_params:   # the unit's parameter shard; the gradient slots are reserved below
                        arena.reserve(u.group, u.shard_numel * es)
                        biggest[id(u.group)] = max(biggest.get(id(u.group), 0), u.padded)
                    else:
                        arena.reserve(u.group, 2 * u.padded * es)
            for key, n in biggest.items():
                arena.reserve(groups[key], 2 * n * es + 1024)
            if self.sharded_params:
                first = next((u for u in self.units if u.size > 1), None)
                if first is not None:   # the first unit's own gradient buffer
                    arena.reserve(first.group, first.padded * es)
            for g in groups.values():
                arena._arena(g)
            self._symm = arena
        except Exception as e:  # noqa: BLE001 - any failure means "use the library path"
            ok, err = False, e
        flag = torch.tensor([1 if ok else 0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 1:
            return True
        self._symm = None
        if self.comm == "nvlink":
            raise RuntimeError(f"fsdp_comm=nvlink requested but symmetric memory setup failed: {err}")
        from torchtitan_b200.utils.logging import logger

        logger.warning(f"symmetric memory unavailable ({err}); FSDP falls back to NCCL collectives")
        self.comm = "nccl"
        return False

    def _materialize_full(self, fqn: str, p, spec: InitSpec) -> torch.Tensor:
        """Local (tensor-parallel sliced) fp32 initial value of parameter ``fqn``."""
        tps = getattr(p, "_tp_slices", None) if not isinstance(p, ParamSlot) else p.tp_slices
        name = self.fqn_prefix + fqn
        if tps is None:
            shape = p.shape
            return materialize_param(shape, spec, self.seed, name, self.device)
        dim, ranges, gshape = tps
        full = materialize_param(gshape, spec, self.seed, name, self.device)
        parts = [full.narrow(dim, a, b - a) for a, b in ranges]
        return torch.cat(parts, dim=dim).contiguous().to(self.device)

    @torch.no_grad()
    def init_weights(self) -> None:
        for u in self.units:
            for s in u.slots:
                full = None
                for slot, pstart, sstart, n in u.slot_pieces():
                    if slot is not s:
                        continue
                    if full is None:
                        full = self._materialize_full(s.fqn, s, s.init).reshape(-1)
                    u.master[sstart:sstart + n].copy_(full[pstart:pstart + n])
                del full
        self.publish_params()
        init_b = getattr(self.model, "init_buffers", None)
        if init_b is not None:
            init_b(self.device)

    @torch.no_grad()
    def publish_params(self) -> None:
        """master shard -> compute-dtype flat_param (own slice) -> all ranks."""
        self.wait_optimizer()
        for u in self.units:
            if u.pool is not None:
                u.param_shard.copy_(u.master)
            else:
                u.shard_view(u.flat_param).copy_(u.master)
        self._all_gather_params()

    def _all_gather_params(self) -> None:
        for u in self.units:
            if u.size > 1 and u.pool is None:
                dist.all_gather_into_tensor(u.flat_param, u.shard_view(u.flat_param), group=u.group)
        self._shards_changed()

    # ------------------------------------------------------------------
    # sharded-parameter layout: gathering units into their slots
    # ------------------------------------------------------------------
    def _shards_changed(self) -> None:
        """Parameter shards were rewritten (optimizer step, checkpoint load): nothing gathered is valid any more,
        and on the NVLink path every rank must have finished writing before anyone pulls."""
        if not self._pools:
            return
        for pool in self._pools.values():
            pool.owner = [None, None]
        if self._symm is not None:
            self._symm.barrier_all()

    def _issue_gather(self, u: FlatUnit) -> None:
        """All-gather ``u`` into its slot on the communication stream (after everything queued so far on the
        compute stream, which includes the last use of the slot's previous occupant)."""
        pool, k = u.pool, u.slot
        cs = self._comm_stream

        def gather():
            if self._symm is not None:
                self._symm.all_gather_shards(u.param_shard, u.gather_dst)
            else:
                dist.all_gather_into_tensor(u.gather_dst, u.param_shard, group=u.group)

        if cs is not None:
            cs.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(cs):
                gather()
                ev = torch.cuda.Event()
                ev.record(cs)
            pool.ready[k] = ev
        else:
            gather()
            pool.ready[k] = None
        pool.owner[k] = u

    def _acquire(self, u: FlatUnit) -> None:
        """Make sure the unit's full parameters are in its slot before the compute stream goes on."""
        pool, k = u.pool, u.slot
        if pool.owner[k] is not u:
            self._issue_gather(u)
        if pool.ready[k] is not None:
            torch.cuda.current_stream(self.device).wait_event(pool.ready[k])

    def _neighbour(self, u: FlatUnit, step: int) -> FlatUnit | None:
        i = self._order.index(u) + step
        return self._order[i] if 0 <= i < len(self._order) else None

    def _pre_forward(self, u: FlatUnit) -> None:
        if u.ready is not None:        # the optimizer step that refreshes this unit may still be running
            torch.cuda.current_stream(self.device).wait_event(u.ready)
            u.ready = None
        if u.pool is None:
            return
        self._acquire(u)
        ev = u.pool.grad_free[u.slot]
        if ev is not None:
            # the fused loss writes the output unit's weight gradients during the forward: the last reduce-scatter
            # out of this gradient slot (an earlier microbatch) must be over
            torch.cuda.current_stream(self.device).wait_event(ev)
        if self._in_backward:      # a recomputed forward inside backward: the backward order prefetches
            return
        nxt = self._neighbour(u, +1)
        if nxt is not None and nxt.pool.owner[nxt.slot] is not nxt:
            self._issue_gather(nxt)                     # overlaps with this unit's forward

    def _pre_backward(self, u: FlatUnit) -> None:
        if u.pool is None:
            return
        self._in_backward = True
        self._acquire(u)
        ev = u.pool.grad_free[u.slot]
        if ev is not None:                               # the reduce-scatter that last read this gradient slot
            torch.cuda.current_stream(self.device).wait_event(ev)
        prv = self._neighbour(u, -1)
        if prv is not None and prv.pool.owner[prv.slot] is not prv:
            self._issue_gather(prv)                     # overlaps with this unit's backward

    # ------------------------------------------------------------------
    # backward-time gradient reduction
    # ------------------------------------------------------------------
    def attach_hooks(self, unit_modules: list[tuple[FlatUnit, nn.Module]]) -> None:
        """Fire the unit's gradient reduction when the gradient reaches the unit's input."""
        for unit, module in unit_modules:
            unit.hooked = True
            module.register_forward_pre_hook(_make_pre_hook(self, unit), with_kwargs=True)
            if unit.pool is not None:
                module.register_forward_hook(_make_post_hook(self, unit))

    def _on_unit_backward_done(self, unit: FlatUnit) -> None:
        self._collect_autograd_grads(unit)
        # sharded layout: the gradient slot is reused by the unit after next, so every microbatch is reduced into
        # the fp32 shard at once, also on pipeline stages (which otherwise keep local gradients until the flush)
        if not self.defer_reduce or (unit.pool is not None and not unit.private_grad):
            self._launch_reduce(unit)

    def _collect_autograd_grads(self, unit: FlatUnit) -> None:
        """Fold gradients delivered through ``.grad`` (ops without direct main_grad writes)."""
        for s in unit.slots:
            p = s.param
            if p.grad is not None:
                if p._main_grad_written:
                    p.main_grad.add_(p.grad)
                else:
                    p.main_grad.copy_(p.grad)
                    p._main_grad_written = True
                p.grad = None

    def _launch_reduce(self, unit: FlatUnit) -> None:
        if unit.pending:
            return
        written = [s.param._main_grad_written for s in unit.slots]
        if not any(written):
            return
        # parameters that received no gradient this pass contribute zeros
        for s, w in zip(unit.slots, written):
            if not w:
                s.param.main_grad.zero_()
        unit.pending = True
        for s in unit.slots:
            s.param._main_grad_written = False
        cs = self._comm_stream
        if cs is not None:
            cs.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(cs):
                self._reduce_unit(unit)
                if unit.pool is not None and not unit.private_grad:
                    ev = torch.cuda.Event()
                    ev.record(cs)
                    unit.pool.grad_free[unit.slot] = ev
        else:
            self._reduce_unit(unit)
        if unit.pool is not None and not unit.private_grad and self.defer_reduce:
            unit.pending = False     # the next microbatch of this pipeline step reduces again

    @torch.no_grad()
    def _reduce_unit(self, u: FlatUnit) -> None:
        tp = self.tp
        if u.rep_reduce_numel and tp is not None and tp.size > 1:
            dist.all_reduce(u.flat_grad[:u.rep_reduce_numel], group=tp.group)
        if u.grad_shard is None:
            # single shard owner, no accumulation: the optimizer reads flat_grad directly
            u.grad_shard_valid = True
            return
        first = not u.grad_shard_valid
        if u.size == 1:
            src = u.flat_grad
            if first:
                u.grad_shard.copy_(src)
            else:
                u.grad_shard.add_(src)
        elif self._symm is not None:
            # a rotating gradient slot is rewritten two units later: its readers are fenced off right here; a unit's
            # own gradient buffer is next written one backward pass later, after the barrier of finish_backward
            slot_backed = u.pool is not None and not u.private_grad
            self._symm.reduce_scatter_accumulate(u.flat_grad, u.grad_shard, u.group, accumulate=not first,
                                                 trailing_barrier=slot_backed)
            self._rs_unfenced = self._rs_unfenced or not slot_backed
        else:
            tmp = self._get_fp32_tmp(u.padded)
            tmp.copy_(u.flat_grad)
            if first:
                dist.reduce_scatter_tensor(u.grad_shard, tmp, group=u.group)
            else:
                out = self._get_fp32_tmp(u.shard_numel, slot=2)
                dist.reduce_scatter_tensor(out, tmp, group=u.group)
                u.grad_shard.add_(out)
        u.grad_shard_valid = True

    def _get_fp32_tmp(self, numel: int, slot: int | None = None) -> torch.Tensor:
        if slot is None:
            slot = self._tmp_idx
            self._tmp_idx ^= 1
        while len(self._fp32_tmp) <= slot:
            self._fp32_tmp.append(torch.empty(0, dtype=torch.float32, device=self.device))
        if self._fp32_tmp[slot].numel() < numel:
            self._fp32_tmp[slot] = torch.empty(numel, dtype=torch.float32, device=self.device)
        return self._fp32_tmp[slot][:numel]

    def finish_backward(self, flush: bool = False) -> None:
        """Reduce units whose input hook did not fire (first unit), then join the comm stream.

        With ``defer_reduce`` (pipeline stages) local gradients keep accumulating over the
        microbatches of a step and nothing is reduced until ``flush=True``."""
        for u in self.units:
            self._collect_autograd_grads(u)
        if self.defer_reduce and not flush:
            return
        for u in self.units:
            self._launch_reduce(u)
        if self._rs_unfenced and self._symm is not None:
            # one barrier for all reduce-scatters of this pass: every rank has finished pulling from every gradient buffer
            cs = self._comm_stream
            with torch.cuda.stream(cs) if cs is not None else contextlib.nullcontext():
                self._symm.barrier_all()
                from . import symm as _symm_mod

                if _symm_mod._CANARY:      # race detection aid: nobody may read these gradients any more
                    for u in self.units:
                        if u.size > 1 and (u.pool is None or u.private_grad):
                            u.flat_grad.fill_(float("nan"))
            self._rs_unfenced = False
        if self._comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
        for u in self.units:
            u.pending = False
        self._callback_queued = False
        self._in_backward = False

    # ------------------------------------------------------------------
    # optimizer-side API
    # ------------------------------------------------------------------
    def _grad_of(self, u: FlatUnit) -> torch.Tensor:
        return u.grad_shard if u.grad_shard is not None else u.shard_view(u.flat_grad)

    @torch.no_grad()
    def finalize_grads(self) -> None:
        """HSDP: sum the reduced shards over the replicate axis."""
        for u in self.units:
            if u.replicate_group is not None and u.grad_shard_valid:
                dist.all_reduce(self._grad_of(u), group=u.replicate_group)

    @torch.no_grad()
    def local_sumsq(self) -> torch.Tensor:
        """``[2]`` fp32: squared norm of this rank's gradient shards, split into the
        tensor-parallel-replicated part and the rest."""
        total = torch.zeros(2, dtype=torch.float32, device=self.device)
        for u in self.units:
            if not u.grad_shard_valid:
                continue
            g = self._grad_of(u)
            lo = u.shard_start
            rep_end = max(0, min(u.rep_numel - lo, u.shard_numel))
            if rep_end > 0:
                optim_ops.sumsq_accumulate(g[:rep_end], total[0:1])
            if rep_end < u.shard_numel:
                optim_ops.sumsq_accumulate(g[rep_end:], total[1:2])
        return total

    def ensure_state(self) -> None:
        self.wait_optimizer()
        for u in self.units:
            if u.exp_avg is None:
                kw = dict(pin_memory=True) if self.offload_optimizer else dict(device=self.device)
                u.exp_avg = torch.zeros(u.shard_numel, dtype=self.state_dtype, **kw)
                u.exp_avg_sq = torch.zeros(u.shard_numel, dtype=self.state_dtype, **kw)

    @torch.no_grad()
    def adamw_step(self, groups: list[dict], grad_scale: torch.Tensor | float = 1.0) -> None:
        """AdamW on every shard; ``groups[i]`` holds lr/betas/eps/weight_decay of param group i."""
        self.ensure_state()
        self.step_count += 1
        step = self.step_count
        fused_ag = self._symm is not None
        if fused_ag and not isinstance(grad_scale, torch.Tensor):
            grad_scale = torch.full((1,), float(grad_scale), dtype=torch.float32, device=self.device)
        if self._overlap_ok(groups):
            self._adamw_step_overlapped(groups, grad_scale, step)
            return
        host_state = None
        for u in self.units:
            if host_state is not None:      # previous unit: updated state back to its pinned host buffers
                self._unstage_state(*host_state)
                host_state = None
            if not u.grad_shard_valid:
                continue
            if self.offload_optimizer:
                host_state = self._stage_state(u)
            g = self._grad_of(u)
            runs = _group_runs(u)
            if any(groups[gi].get("optimizer_name") == "DistMuon" for gi, _a, _b in runs) or any(
                    groups[s.group_idx].get("optimizer_name") == "DistMuon" for s in u.slots):
                # Muon needs whole matrices: owner-computes over the unit's group (parallel/muon.py)
                from .muon import muon_unit_step

                if u.pool is not None:
                    raise NotImplementedError("DistMuon needs the resident parameter layout "
                                              "(parallelism.fsdp_reshard_after_forward = never)")
                muon_unit_step(self, u, groups, runs, step, grad_scale)
                if fused_ag and u.size > 1:
                    dist.all_gather_into_tensor(u.flat_param, u.shard_view(u.flat_param).clone(), group=u.group)
                u.grad_shard_valid = False
                continue
            if fused_ag and u.size > 1 and u.pool is None:
                # update + all-gather in one kernel: refreshed weights are stored to every peer
                self._symm.adamw_allgather(u, _group_runs(u), groups, step, grad_scale.reshape(1), g)
                u.grad_shard_valid = False
                continue
            lowp = u.param_shard if u.pool is not None else u.shard_view(u.flat_param)
            for gi, a, b in _group_runs(u):
                h = groups[gi]
                optim_ops.adamw_(
                    u.master[a:b], g[a:b], u.exp_avg[a:b], u.exp_avg_sq[a:b], lowp[a:b],
                    lr=h["lr"], beta1=h["betas"][0], beta2=h["betas"][1], eps=h["eps"],
                    weight_decay=h["weight_decay"], step=step, grad_scale=grad_scale,
                )
            u.grad_shard_valid = False
        if host_state is not None:
            self._unstage_state(*host_state)
        if self.offload_optimizer:
            torch.cuda.current_stream(self.device).synchronize()   # host buffers are complete before anyone reads them
        if fused_ag:
            if not self._pools:
                self._symm.barrier_all()  # peers' stores into our parameter buffers have landed
            else:
                self._shards_changed()    # (includes the barrier)
        else:
            self._all_gather_params()

    # -- optimizer overlapped with the next forward ---------------------------------------
    def _overlap_ok(self, groups: list[dict]) -> bool:
        """The update (and weight refresh) of unit k only has to be finished when the next forward reaches unit k.
        Resident layout on CUDA, plain AdamW, state on the device; ``TB200_OVERLAP_OPTIMIZER=0`` switches it off."""
        import os

        return (self._comm_stream is not None and not self._pools and not self.offload_optimizer
                and os.environ.get("TB200_OVERLAP_OPTIMIZER", "1") != "0"
                and not any(g.get("optimizer_name") == "DistMuon" for g in groups))

    def _adamw_step_overlapped(self, groups: list[dict], grad_scale, step: int) -> None:
        """Units are updated in forward order on the communication stream; each unit records an event once its
        refreshed weights are in place on every rank (after the unit's flag barrier or NCCL all-gather), and the
        unit's forward pre-hook makes the compute stream wait for exactly that event.  The rest of the optimizer
        therefore runs under the first layers of the next forward."""
        cs = self._comm_stream
        main = torch.cuda.current_stream(self.device)
        fused_ag = self._symm is not None
        if isinstance(grad_scale, torch.Tensor):
            grad_scale.record_stream(cs)
        cs.wait_stream(main)
        with torch.cuda.stream(cs):
            for u in self.units:
                if u.grad_shard_valid:
                    g = self._grad_of(u)
                    if fused_ag and u.size > 1:
                        self._symm.adamw_allgather(u, _group_runs(u), groups, step, grad_scale.reshape(1), g)
                        self._symm.barrier_group(u.group)      # every rank's stores into this unit have landed
                    else:
                        lowp = u.shard_view(u.flat_param)
                        for gi, a, b in _group_runs(u):
                            h = groups[gi]
                            optim_ops.adamw_(
                                u.master[a:b], g[a:b], u.exp_avg[a:b], u.exp_avg_sq[a:b], lowp[a:b],
                                lr=h["lr"], beta1=h["betas"][0], beta2=h["betas"][1], eps=h["eps"],
                                weight_decay=h["weight_decay"], step=step, grad_scale=grad_scale,
                            )
                        if u.size > 1:
                            dist.all_gather_into_tensor(u.flat_param, lowp, group=u.group)
                    u.grad_shard_valid = False
                ev = torch.cuda.Event()
                ev.record(cs)
                u.ready = ev
        for u in self.units:
            if not u.hooked:          # no forward hook will wait for it
                main.wait_event(u.ready)
                u.ready = None
        self._optimizer_inflight = True

    def wait_optimizer(self) -> None:
        """Make the current stream wait for an optimizer step that is still running on the communication stream
        (before anything outside the units' forward hooks reads parameters or optimizer state)."""
        if self._optimizer_inflight:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
            for u in self.units:
                u.ready = None
            self._optimizer_inflight = False

    def _stage_state(self, u: FlatUnit):
        """Offloaded optimizer state of one unit -> device copies (the unit's attributes point at
        them while it is updated)."""
        host = (u.master, u.exp_avg, u.exp_avg_sq)
        u.master, u.exp_avg, u.exp_avg_sq = (t.to(self.device, non_blocking=True) for t in host)
        return u, host

    def _unstage_state(self, u: FlatUnit, host) -> None:
        for h, d in zip(host, (u.master, u.exp_avg, u.exp_avg_sq)):
            h.copy_(d, non_blocking=True)
        u.master, u.exp_avg, u.exp_avg_sq = host

    def check_status(self) -> None:
        """Raise if a bounded device-side wait expired (host sync; call at logging points)."""
        if self._symm is not None:
            self._symm.check_status()

    def zero_grad(self) -> None:
        for u in self.units:
            u.grad_shard_valid = False
            u.pending = False
            for s in u.slots:
                s.param._main_grad_written = False
                s.param.grad = None

    # ------------------------------------------------------------------
    # parameter-group assignment and state export
    # ------------------------------------------------------------------
    def assign_groups(self, patterns: list[str]) -> list[list[str]]:
        """First matching regex wins; unmatched parameters go to the last (default) group."""
        compiled = [re.compile(p) for p in patterns]
        members: list[list[str]] = [[] for _ in range(len(patterns) + 1)]
        for u in self.units:
            for s in u.slots:
                gi = len(patterns)
                for i, rx in enumerate(compiled):
                    if rx.search(s.fqn):
                        gi = i
                        break
                s.group_idx = gi
                members[gi].append(s.fqn)
        return members

    def named_slots(self) -> Iterable[tuple[FlatUnit, ParamSlot]]:
        for u in self.units:
            for s in u.slots:
                yield u, s

    def param_layout(self) -> str:
        """One-line description of where parameters and gradients live (reported by the benchmark)."""
        if all(u.size == 1 for u in self.units):
            return "single rank: bf16 parameters and gradients, fp32 master weights and moments"
        if self._pools:
            return ("bf16 parameters sharded 1/N between uses (two gather slots and two gradient slots per group, next "
                    "unit prefetched on the communication stream), fp32 master weights and moments sharded 1/N")
        return ("bf16 parameters and gradients replicated on every rank (resident, refreshed once per step by the "
                "optimizer kernel), fp32 master weights and moments sharded 1/N")

    def memory_summary(self) -> dict[str, float]:
        gib = 1 << 30
        tot = {"flat_param": 0, "flat_grad": 0, "master": 0, "grad_shard": 0, "opt_state": 0}
        for pool in self._pools.values():
            tot["flat_param"] += sum(t.numel() * t.element_size() for t in pool.param)
            tot["flat_grad"] += sum(t.numel() * t.element_size() for t in pool.grad)
        for u in self.units:
            if u.pool is not None:
                tot["flat_param"] += u.param_shard.numel() * u.param_shard.element_size()
            else:
                tot["flat_param"] += u.flat_param.numel() * u.flat_param.element_size()
                tot["flat_grad"] += u.flat_grad.numel() * u.flat_grad.element_size()
            tot["master"] += u.master.numel() * 4
            if u.grad_shard is not None:
                tot["grad_shard"] += u.grad_shard.numel() * 4
            if u.exp_avg is not None:
                tot["opt_state"] += 2 * u.exp_avg.numel() * u.exp_avg.element_size()
        return {k: v / gib for k, v in tot.items()}


class _SlotPool:
    """Two rotating full-size parameter buffers and two gradient buffers shared by the units of one sharding
    group (sharded-parameter layout).  ``owner[k]`` is the unit whose gathered parameters slot ``k`` holds,
    ``ready[k]`` the event of that gather, ``grad_free[k]`` the event of the last reduce-scatter out of
    gradient slot ``k``."""

    def __init__(self, param: list[torch.Tensor], grad: list[torch.Tensor]):
        self.param, self.grad = param, grad
        self.owner: list = [None, None]
        self.ready: list = [None, None]
        self.grad_free: list = [None, None]


def _alias(t: torch.Tensor, numel: int) -> torch.Tensor:
    """A fresh tensor over the first ``numel`` elements of ``t``'s storage.  It shares memory but not the
    autograd version counter, so gathering into it does not invalidate tensors that autograd saved from a
    sibling alias (the values are the same before and after a re-gather)."""
    out = torch.empty(0, dtype=t.dtype, device=t.device)
    out.set_(t.untyped_storage(), t.storage_offset(), (numel,), (1,))
    return out


def _group_runs(u: FlatUnit):
    """Maximal runs ``(group_idx, shard_lo, shard_hi)`` of this rank's shard with one param group.
    A run extends to the start of the next run (or the end of the shard), so alignment padding
    rides along and every boundary is a multiple of 8 elements."""
    starts: list[list[int]] = []
    for slot, _pstart, sstart, _n in u.slot_pieces():
        if not starts or starts[-1][0] != slot.group_idx:
            starts.append([slot.group_idx, sstart])
    runs = []
    for i, (g, a) in enumerate(starts):
        b = starts[i + 1][1] if i + 1 < len(starts) else u.shard_numel
        runs.append((g, 0 if i == 0 else a, b))
    return runs


def _swap_parameters(model: nn.Module, replaced: dict[int, nn.Parameter]) -> None:
    for mod in model.modules():
        for name, p in list(mod._parameters.items()):
            if p is not None and id(p) in replaced:
                mod._parameters[name] = replaced[id(p)]


class _UnitBackwardEnd(torch.autograd.Function):
    """Identity on the unit's inputs whose backward marks the end of the unit's backward."""

    @staticmethod
    def forward(ctx, engine, unit, *tensors):
        ctx.engine, ctx.unit = engine, unit
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        ctx.engine._on_unit_backward_done(ctx.unit)
        return (None, None) + grads


class _UnitBackwardStart(torch.autograd.Function):
    """Identity on the unit's outputs whose backward re-gathers the unit's parameters (sharded layout)."""

    @staticmethod
    def forward(ctx, engine, unit, *tensors):
        ctx.engine, ctx.unit = engine, unit
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        ctx.engine._pre_backward(ctx.unit)
        return (None, None) + grads


def _make_post_hook(engine: ShardedModel, unit: FlatUnit):
    def hook(module, args, output):
        if not torch.is_grad_enabled():
            return None
        if isinstance(output, torch.Tensor):
            if not output.requires_grad:
                return None
            return _UnitBackwardStart.apply(engine, unit, output)[0]
        if isinstance(output, tuple):
            idx = [i for i, o in enumerate(output) if isinstance(o, torch.Tensor) and o.requires_grad]
            if not idx:
                return None
            outs = _UnitBackwardStart.apply(engine, unit, *[output[i] for i in idx])
            res = list(output)
            for i, o in zip(idx, outs):
                res[i] = o
            return tuple(res)
        return None

    return hook


def _make_pre_hook(engine: ShardedModel, unit: FlatUnit):
    def hook(module, args, kwargs):
        engine._pre_forward(unit)
        if not torch.is_grad_enabled():
            return None
        if not engine._callback_queued:
            # runs once per backward pass, after the last autograd node
            engine._callback_queued = True
        idx = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor) and a.requires_grad]
        if not idx:
            return None
        outs = _UnitBackwardEnd.apply(engine, unit, *[args[i] for i in idx])
        args = list(args)
        for i, o in zip(idx, outs):
            args[i] = o
        return tuple(args), kwargs

    return hook
