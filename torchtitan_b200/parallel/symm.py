"""Symmetric-memory arena and the NVLink collectives built on it.

One arena per process group: a single symmetric allocation (same size and layout on
every rank, obtained from ``torch.distributed._symmetric_memory``) from which the engine
carves its flat parameter / gradient buffers, plus a small symmetric flag array for
barriers.  Every rank knows every peer's base pointer, so our kernels address peer
memory directly with ``ld/st.global`` over NVLink / NVSwitch (parity with the reference's
use of symmetric memory for FSDP and MinimalAsyncEP, torchtitan/distributed/fsdp.py:102-109,
torchtitan/distributed/minimal_async_ep/api.py:174-295, re-designed around in-kernel
transfers).

Synchronisation is a flag barrier with monotonically increasing epochs.  The epoch lives in
device memory and is advanced by the barrier kernel itself, so a barrier captured into a CUDA
graph publishes a new epoch on every replay.  Waits are bounded (``TB200_SYMM_TIMEOUT_S``,
default 30 s): on expiry the kernel sets a bit in a status word and returns.  Every arena
registers its status word with :class:`StatusMonitor`; the trainer polls the monitor every step
(an asynchronous copy to pinned memory, checked one step later, no synchronisation) and raises
when any word is non-zero.  Nothing traps the device.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from torchtitan_b200.ops import ext
from torchtitan_b200.ops.functional import _count

__all__ = ["SymmetricArena", "StatusMonitor", "status_monitor", "symm_available"]


class StatusMonitor:
    """Collects the status words of every bounded-wait path and checks them without stalling the GPU.

    ``poll()`` queues a device-to-pinned-host copy of all registered words on the current stream and
    examines the copy queued by the previous ``poll()`` if its event has completed (it always has
    one step later); ``check()`` synchronises and examines the current values.  Both raise
    ``RuntimeError`` naming the path whose wait expired."""

    def __init__(self):
        self._words: list[tuple[str, torch.Tensor]] = []
        self._inflight: tuple | None = None
        self.tolerated = 0      # status bits that are logged instead of raised (8: dropped expert-parallel rows)
        self.tolerated_seen = 0

    def register(self, name: str, word: torch.Tensor) -> None:
        self._words.append((name, word))

    def clear(self) -> None:
        self._words.clear()
        self._inflight = None
        self.tolerated = 0
        self.tolerated_seen = 0

    # bits of a status word (ops/csrc/common.cuh, moe.cu)
    _BITS = ((1, "a RoPE position outside the table"), (2, "a label outside the vocabulary"),
             (4, "a bounded device wait expired: a peer did not arrive within the timeout (TB200_SYMM_TIMEOUT_S), the "
                 "data exchanged in that step is incomplete"),
             (8, "an expert-parallel receive buffer overflowed: more rows were routed to this rank than "
                 "parallelism.ep_capacity_factor allows, the rows that did not fit were dropped (raise the factor, or "
                 "set it to 0 for the worst-case capacity)"))

    def _raise_if_set(self, values: list[int], names: list[str]) -> None:
        if self.tolerated and any(v & self.tolerated for v in values):
            self.tolerated_seen += 1
            if self.tolerated_seen in (1, 10, 100) or self.tolerated_seen % 1000 == 0:
                from torchtitan_b200.utils.logging import logger

                logger.warning("tolerated device status (seen %d times): %s", self.tolerated_seen, "; ".join(
                    f"{n}: " + ", ".join(t for b, t in self._BITS if v & b & self.tolerated) for n, v in zip(names, values)
                    if v & self.tolerated))
            for (_, w), v in zip(self._words, values):
                if v & self.tolerated and not v & ~self.tolerated:
                    w.zero_()
            values = [v & ~self.tolerated for v in values]
        bad = [(n, v) for n, v in zip(names, values) if v]
        if bad:
            for _, w in self._words:
                w.zero_()
            desc = "; ".join(f"{n} (status {v:#x}): " + ", ".join(text for bit, text in self._BITS if v & bit)
                             for n, v in bad)
            raise RuntimeError(f"device status set in {desc}; training stops here")

    def poll(self) -> None:
        if not self._words:
            return
        if self._inflight is not None:
            host, ev, names = self._inflight
            if ev is None or ev.query():
                self._inflight = None
                self._raise_if_set([int(x) for x in host.tolist()], names)
            else:
                return   # the previous copy has not landed yet: look again next step
        words = [w.reshape(-1)[:1] for _, w in self._words]
        names = [n for n, _ in self._words]
        dev = torch.cat(words)
        if dev.is_cuda:
            host = torch.empty(dev.numel(), dtype=dev.dtype, pin_memory=True)
            host.copy_(dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            host, ev = dev.clone(), None
        self._inflight = (host, ev, names)

    def check(self) -> None:
        if not self._words:
            return
        self._inflight = None
        vals = [int(w.reshape(-1)[0].item()) for _, w in self._words]
        self._raise_if_set(vals, [n for n, _ in self._words])


status_monitor = StatusMonitor()

_FLAG_SLOTS = 64
# TB200_SYMM_CANARY=1: symmetric gradient buffers are filled with NaN once every rank has finished reading them
_CANARY = os.environ.get("TB200_SYMM_CANARY", "0") == "1"


def symm_available() -> bool:
    try:
        import torch.distributed._symmetric_memory  # noqa: F401

        return torch.cuda.is_available()
    except Exception:
        return False


class _GroupArena:
    def __init__(self, group, device: torch.device, nbytes: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        gname = group.group_name
        try:
            symm_mem.enable_symm_mem_for_group(gname)
        except Exception:
            pass
        total = nbytes + 4096
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, gname)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # NVSwitch multicast address of the same buffer (0 when the fabric or the driver has none);
        # TB200_MULTICAST=0 keeps every store on plain peer addresses
        self.mc_base = 0
        if os.environ.get("TB200_MULTICAST", "1") != "0":
            try:
                self.mc_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            except Exception:
                self.mc_base = 0
            if self.rank == 0:
                from torchtitan_b200.utils.logging import logger

                logger.info(f"symmetric arena of group {gname}: multicast stores {'on' if self.mc_base else 'unavailable'}")
        self.flags = symm_mem.empty(_FLAG_SLOTS * self.size, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flag_handle = symm_mem.rendezvous(self.flags, gname)
        self.flag_ptrs = [int(p) for p in self.flag_handle.buffer_ptrs]
        self.cursor = 0
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)   # advanced by the barrier kernel
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        status_monitor.register(f"symmetric arena of group {gname}", self.status)
        clock_hz = 1e3 * float(getattr(torch.cuda.get_device_properties(device), "clock_rate", 1.9e6) or 1.9e6)
        self.max_cycles = int(float(os.environ.get("TB200_SYMM_TIMEOUT_S", "30")) * clock_hz)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def carve(self, numel: int, dtype: torch.dtype) -> tuple[torch.Tensor, int]:
        es = torch.empty(0, dtype=dtype).element_size()
        off = (self.cursor + 255) // 256 * 256
        nbytes = numel * es
        if off + nbytes > self.buf.numel():
            raise RuntimeError("symmetric arena exhausted")
        self.cursor = off + nbytes
        # A fresh tensor over the same storage (not an autograd view of ``buf``): carved buffers
        # must not share a version counter, or writing gradients would invalidate tensors that
        # autograd saved from the parameter buffer.
        t = torch.empty(0, dtype=dtype, device=self.device)
        t.set_(self.buf.untyped_storage(), (self.buf.storage_offset() + off) // es, (numel,), (1,))
        return t, off

    def barrier(self, bump: torch.Tensor | None = None) -> None:
        """Cross-rank barrier on the current stream (bounded wait).  ``bump``: an int32[1] device
        counter advanced by one in the same launch."""
        _count()
        ext.require().symm_barrier(self.flag_ptrs, self.rank, self.epoch, self.status, self.max_cycles, bump)


class SymmetricArena:
    """Per-process collection of group arenas; the engine's entry point to the NVLink path."""

    def __init__(self, pdims, device: torch.device):
        self.pdims = pdims
        self.device = device
        self._arenas: dict[int, _GroupArena] = {}
        self._offsets: dict[int, tuple[_GroupArena, int]] = {}
        self._reserved: dict[int, int] = {}

    def reserve(self, group, nbytes: int) -> None:
        """Declare how many bytes will be carved for ``group`` (call before the first alloc)."""
        self._reserved[id(group)] = self._reserved.get(id(group), 0) + nbytes + 512

    def _arena(self, group) -> _GroupArena:
        key = id(group)
        if key not in self._arenas:
            if key not in self._reserved:
                raise RuntimeError("SymmetricArena.reserve must be called before alloc")
            self._arenas[key] = _GroupArena(group, self.device, self._reserved[key])
        return self._arenas[key]

    def alloc(self, numel: int, dtype: torch.dtype, group, tag: str = "") -> torch.Tensor:
        arena = self._arena(group)
        t, off = arena.carve(numel, dtype)
        self._offsets[t.data_ptr()] = (arena, off)
        return t

    def _locate(self, t: torch.Tensor) -> tuple[_GroupArena, int]:
        arena, off = self._offsets[t.data_ptr()]
        return arena, off

    def peer_ptrs(self, t: torch.Tensor) -> tuple[_GroupArena, list[int]]:
        arena, off = self._locate(t)
        return arena, [b + off for b in arena.base_ptrs]

    # -- collectives -----------------------------------------------------------
    def reduce_scatter_accumulate(self, flat_grad: torch.Tensor, grad_shard: torch.Tensor, group,
                                  accumulate: bool, trailing_barrier: bool = True) -> None:
        """``grad_shard (+)= sum over ranks of flat_grad[my slice]`` by pulling from peers.

        The barrier in front makes every rank's local gradients complete.  A second barrier after the pull keeps a
        rank from overwriting a gradient buffer that a peer still reads; the caller may leave it out when a later
        barrier of the same arena on the same stream is certain to follow before the buffer is written again."""
        arena, ptrs = self.peer_ptrs(flat_grad)
        arena.barrier()
        _count()
        ext.require().reduce_scatter_pull(ptrs, arena.rank, arena.rank * grad_shard.numel(), grad_shard,
                                          flat_grad.dtype == torch.bfloat16, accumulate)
        if trailing_barrier:
            arena.barrier()
            if _CANARY:
                # race detection aid: after the fence nobody may read these gradients again; poison them so that a
                # stale read (a missing barrier, a wrong buffer) shows up as NaN in the loss instead of going unnoticed
                flat_grad.fill_(float("nan"))

    def adamw_allgather(self, unit, runs, groups, step: int, grad_scale: torch.Tensor, grad: torch.Tensor) -> None:
        """AdamW on this rank's shard with the weight all-gather fused in (peer stores)."""
        arena, ptrs = self.peer_ptrs(unit.flat_param)
        bf16 = unit.flat_param.dtype == torch.bfloat16
        ops = ext.require()
        for gi, a, b in runs:
            h = groups[gi]
            b1, b2 = h["betas"]
            _count()
            mc = 0
            if arena.mc_base:
                mc = arena.mc_base + (ptrs[arena.rank] - arena.base_ptrs[arena.rank])   # same offset inside the arena
            ops.adamw_allgather_(unit.master[a:b], grad[a:b], unit.exp_avg[a:b], unit.exp_avg_sq[a:b], ptrs,
                                 arena.rank, unit.shard_start + a, bf16, mc, grad_scale, float(h["lr"]), float(b1),
                                 float(b2), float(h["eps"]), float(h["weight_decay"]), 1.0 - b1 ** step,
                                 1.0 - b2 ** step)

    def all_gather_shards(self, shard: torch.Tensor, out: torch.Tensor) -> None:
        """``out[r * n:(r + 1) * n] = rank r's shard`` for every rank, by 16-byte peer loads (``shard`` is a
        symmetric allocation, ``out`` local).  No barrier: the caller guarantees that no rank is writing its
        shard (parameter shards change only inside the optimizer step, which ends with a barrier)."""
        arena, ptrs = self.peer_ptrs(shard)
        nbytes = shard.numel() * shard.element_size()
        _count()
        ext.require().all_gather_pull(ptrs, arena.rank, nbytes, out)

    def barrier_group(self, group) -> None:
        self._arenas[id(group)].barrier()

    def barrier_all(self) -> None:
        for arena in self._arenas.values():
            arena.barrier()

    def check_status(self) -> None:
        """Host-side check of the device status words (synchronises)."""
        for arena in self._arenas.values():
            v = int(arena.status.item())
            if v:
                arena.status.zero_()
                raise RuntimeError(
                    f"a bounded device wait expired (status {v:#x}) in the NVLink path of group "
                    f"{arena.group.group_name}: a peer did not arrive within the timeout")
