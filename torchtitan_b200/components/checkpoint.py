"""Checkpointing in the ``torch.distributed.checkpoint`` (DCP) file format.

Layout on disk: ``<dump_folder>/<folder>/step-<N>/`` with DCP ``.metadata`` and
``__<rank>_<i>.distcp`` files.  The saved dict has the model tensors flattened at
top level under their un-fused names (``layers.0.attention.qkv_linear.wq.weight``),
plus ``optimizer`` (``state.<fqn>.exp_avg`` ...), ``lr_scheduler``, ``dataloader``
and ``train_state`` -- the layout of torchtitan/components/checkpointer/dcp.py:172-180,
717-738, so model-only checkpoints interoperate with the reference / torchtune.

Sharding.  The engine shards flat buffers by offset, so a rank owns an arbitrary
flat interval of each parameter.  ``ShardedEntry`` describes that interval as
rectangles in *global* tensor coordinates (after undoing fused-row and
tensor-parallel slicing); the planners below turn the rectangles into ordinary DCP
chunks.  Because files only contain global-coordinate chunks, a checkpoint can be
loaded under any other parallel layout, and checkpoints written by FSDP2/DTensor
load here.

Policies (parity: checkpointer/base.py:187-398, dcp.py:401-853): interval / first
step / last step saves, model-only last save with ``export_dtype``, Hugging Face
safetensors export and import through the model's adapter, ``keep_latest_k`` purge
in a background thread, ``load_step``, ``exclude_from_loading``, ``load_only``,
``initial_load_path``, seed checkpoints, and asynchronous saves (device->pinned-host
staging on a side stream, then ``dcp.save`` from a thread over a gloo group).
"""

from __future__ import annotations

import enum
import os
import queue
import re
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Literal

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
from torch.distributed.checkpoint.metadata import (
    ChunkStorageMetadata, MetadataIndex, TensorProperties, TensorStorageMetadata,
)
from torch.distributed.checkpoint.planner import (
    LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType,
)
from torch.distributed.checkpoint.planner_helpers import create_read_items_for_chunk_list

from torchtitan_b200.config import Configurable
from torchtitan_b200.models.common.module import iter_checkpoint_slices
from torchtitan_b200.utils import filesystem as fsys
from torchtitan_b200.utils import structured_logger as sl
from torchtitan_b200.utils.logging import logger

__all__ = ["CheckpointManager", "ShardedEntry", "AsyncMode", "engine_model_state", "engine_optimizer_state",
           "load_engine_optimizer_state", "ChunkSavePlanner", "ChunkLoadPlanner", "flat_interval_to_boxes"]

MODEL, OPTIMIZER, LR_SCHEDULER, DATALOADER, TRAIN_STATE = "model", "optimizer", "lr_scheduler", "dataloader", "train_state"


class AsyncMode(str, enum.Enum):
    DISABLED = "disabled"
    ASYNC = "async"
    ASYNC_WITH_PINNED_MEM = "async_with_pinned_mem"


# ----------------------------------------------------------------------
# chunk geometry
# ----------------------------------------------------------------------
@dataclass
class ShardedEntry:
    """This rank's pieces of one global tensor: ``chunks = [(offsets, sizes, tensor)]``."""

    global_shape: tuple[int, ...]
    dtype: torch.dtype
    chunks: list[tuple[tuple[int, ...], tuple[int, ...], torch.Tensor]] = field(default_factory=list)


def flat_interval_to_boxes(shape: tuple[int, ...], start: int, length: int):
    """Split the flat interval ``[start, start+length)`` of a row-major tensor of ``shape``
    into axis-aligned boxes ``(offsets, sizes, flat_offset)``; ``flat_offset`` is the
    position of the box inside the interval (each box is contiguous in memory)."""
    if length <= 0:
        return []
    if len(shape) <= 1:
        return [((start,), (length,), 0)]
    inner = 1
    for s in shape[1:]:
        inner *= s
    out = []
    pos, end = start, start + length
    r, c = divmod(pos, inner)
    if c != 0:
        n = min(inner - c, end - pos)
        for o, z, f in flat_interval_to_boxes(tuple(shape[1:]), c, n):
            out.append(((r,) + o, (1,) + z, (pos - start) + f))
        pos += n
    full = (end - pos) // inner
    if full > 0:
        out.append(((pos // inner,) + (0,) * (len(shape) - 1), (full,) + tuple(shape[1:]), pos - start))
        pos += full * inner
    if pos < end:
        r = pos // inner
        for o, z, f in flat_interval_to_boxes(tuple(shape[1:]), 0, end - pos):
            out.append(((r,) + o, (1,) + z, (pos - start) + f))
    return out


flat_interval_to_rects = flat_interval_to_boxes


def _row_maps(slot, slices_of_param):
    """``[(local_row0, local_row1, ckpt_name, ckpt_row0, ckpt_shape)]``: how the local
    (parallel-sliced, fused) leading-dim rows of a parameter map onto checkpoint tensors."""
    shape = slot.shape if len(slot.shape) else (1,)
    tps = slot.tp_slices
    rows = shape[0]
    if tps is not None and tps[0] == 0:
        segs, base = [], 0
        for a, b in tps[1]:
            segs.append((base, base + (b - a), a))
            base += b - a
        gshape = tuple(tps[2])
    else:
        segs = [(0, rows, 0)]
        gshape = tuple(tps[2]) if tps is not None else tuple(shape)
    pieces = slices_of_param or [(slot.fqn, 0, gshape[0])]
    out = []
    for l0, l1, g0 in segs:
        for name, p0, p1 in pieces:
            lo, hi = max(g0, p0), min(g0 + (l1 - l0), p1)
            if lo < hi:
                out.append((l0 + (lo - g0), l0 + (hi - g0), name, lo - p0, (p1 - p0,) + gshape[1:]))
    return out


def _entries_for_flat(engine, pick_flat, dtype=None, key_fmt="{}") -> dict[str, ShardedEntry]:
    """Build ``{checkpoint_fqn: ShardedEntry}`` from per-unit flat shard tensors."""
    if hasattr(engine, "wait_optimizer"):
        engine.wait_optimizer()        # an optimizer step overlapped with the next forward must have finished
    slices = _global_slices(engine)
    out: dict[str, ShardedEntry] = {}
    for u in engine.units:
        flat = pick_flat(u)
        if flat is None:
            continue
        for slot, pstart, sstart, n in u.slot_pieces():
            shape = slot.shape if len(slot.shape) else (1,)
            inner_off = [0] * len(shape)
            if slot.tp_slices is not None and slot.tp_slices[0] > 0:
                inner_off[slot.tp_slices[0]] = slot.tp_slices[1][0][0]
            maps = _row_maps(slot, slices.get(slot.fqn, []))
            for offs, sizes, foff in flat_interval_to_boxes(tuple(shape), pstart, n):
                numel = 1
                for z in sizes:
                    numel *= z
                src = flat[sstart + foff: sstart + foff + numel]
                r0, nr = offs[0], sizes[0]
                per_row = numel // nr
                for l0, l1, name, g0, cshape in maps:
                    lo, hi = max(r0, l0), min(r0 + nr, l1)
                    if lo >= hi:
                        continue
                    piece = src[(lo - r0) * per_row:(hi - r0) * per_row]
                    goffs = (g0 + (lo - l0),) + tuple(o + io for o, io in zip(offs[1:], inner_off[1:]))
                    gsizes = (hi - lo,) + tuple(sizes[1:])
                    key = key_fmt.format(name)
                    ent = out.get(key)
                    if ent is None:
                        ent = out[key] = ShardedEntry(tuple(cshape), dtype or flat.dtype)
                    ent.chunks.append((goffs, gsizes, piece.view(gsizes)))
    return out


def _global_slices(engine) -> dict[str, list[tuple[str, int, int]]]:
    """Fused-parameter row pieces in *global* (un-tp-sliced) rows."""
    local = dict(iter_checkpoint_slices(engine.model))
    out = {}
    tp = engine.tp
    for fqn, pieces in local.items():
        if tp is None or tp.size == 1:
            out[fqn] = pieces
        else:
            base = 0
            conv = []
            for name, a, b in pieces:  # local block sizes -> global block ranges
                g = (b - a) * tp.size
                conv.append((name, base, base + g))
                base += g
            out[fqn] = conv
    return out


def engine_model_state(engine, dtype: torch.dtype | None = None) -> dict[str, ShardedEntry]:
    return _entries_for_flat(engine, lambda u: u.master, dtype)


_GROUP_KEYS = ("lr", "betas", "eps", "weight_decay", "initial_lr")
# torch.optim.AdamW fields that the reference's flattened optimizer dict also carries; constant here
_GROUP_CONSTANTS = {"amsgrad": False, "maximize": False, "foreach": None, "capturable": False, "differentiable": False,
                    "fused": True}


def _checkpoint_names(engine) -> list[tuple[str, int]]:
    """``(checkpoint fqn, optimizer group index)`` of every parameter of the engine, whichever rank holds its rows."""
    slices = _global_slices(engine)
    out = []
    for u in engine.units:
        for slot in u.slots:
            for _l0, _l1, name, _g0, _cshape in _row_maps(slot, slices.get(slot.fqn, [])):
                out.append((name, slot.group_idx))
    return out


def engine_optimizer_state(engine, param_groups: list[dict]) -> dict[str, Any]:
    """The optimizer state in the key scheme of the reference's flattened DCP optimizer dict
    (``get_optimizer_state_dict(..., flatten_optimizer_state_dict=True)``, torchtitan/components/optimizer.py):
    ``state.{fqn}.exp_avg`` / ``exp_avg_sq`` / ``step`` and ``param_groups.{fqn}.{field}`` per parameter."""
    engine.ensure_state()
    out: dict[str, Any] = {}
    out.update(_entries_for_flat(engine, lambda u: u.exp_avg, key_fmt="state.{}.exp_avg"))
    out.update(_entries_for_flat(engine, lambda u: u.exp_avg_sq, key_fmt="state.{}.exp_avg_sq"))
    step = torch.tensor(float(engine.step_count))
    for name, gi in _checkpoint_names(engine):
        out[f"state.{name}.step"] = step.clone()
        g = param_groups[gi] if gi < len(param_groups) else param_groups[-1]
        for k in _GROUP_KEYS:
            if k in g:
                out[f"param_groups.{name}.{k}"] = list(g[k]) if isinstance(g[k], tuple) else g[k]
        for k, v in _GROUP_CONSTANTS.items():
            out[f"param_groups.{name}.{k}"] = v
    return out


def load_engine_optimizer_state(engine, sd: dict[str, Any], param_groups: list[dict]) -> None:
    """Moments were loaded in place through the ShardedEntry views; the step and the group fields come from the
    per-parameter keys (or from the single ``step`` / index-keyed ``param_groups.{i}.*`` of earlier checkpoints)."""
    names = _checkpoint_names(engine)
    step = sd.get("step")
    for name, _ in names:
        if f"state.{name}.step" in sd:
            step = sd[f"state.{name}.step"]
            break
    if step is not None:
        engine.step_count = int(step.item() if isinstance(step, torch.Tensor) else step)
    seen: set[int] = set()
    for name, gi in names:
        if gi in seen or gi >= len(param_groups):
            continue
        g = param_groups[gi]
        for k in _GROUP_KEYS:
            key = f"param_groups.{name}.{k}"
            if key in sd:
                g[k] = tuple(sd[key]) if k == "betas" else sd[key]
                seen.add(gi)
    for i, g in enumerate(param_groups):
        for k in _GROUP_KEYS:
            key = f"param_groups.{i}.{k}"
            if i not in seen and key in sd:
                g[k] = tuple(sd[key]) if k == "betas" else sd[key]


# ----------------------------------------------------------------------
# DCP planners that understand ShardedEntry
# ----------------------------------------------------------------------
def _flatten(prefix: str, obj: Any, out: dict[str, Any]) -> None:
    if isinstance(obj, dict):
        for k, v in obj.items():
            _flatten(f"{prefix}.{k}" if prefix else str(k), v, out)
    else:
        out[prefix] = obj


class ChunkSavePlanner(DefaultSavePlanner):
    def __init__(self, writer_rank_filter: bool = True, **kw):
        super().__init__(flatten_state_dict=False, dedup_save_to_lowest_rank=True, **kw)
        self._entries: dict[str, ShardedEntry] = {}
        self._write_sharded = writer_rank_filter

    def set_up_planner(self, state_dict, storage_meta=None, is_coordinator=False):
        flat: dict[str, Any] = {}
        _flatten("", state_dict, flat)
        self._entries = {k: v for k, v in flat.items() if isinstance(v, ShardedEntry)}
        plain = {k: v for k, v in flat.items() if not isinstance(v, ShardedEntry)}
        super().set_up_planner(plain, storage_meta, is_coordinator)

    def create_local_plan(self) -> SavePlan:
        plan = super().create_local_plan()
        items = list(plan.items)
        if self._write_sharded:
            for fqn, ent in self._entries.items():
                for offsets, sizes, t in ent.chunks:
                    items.append(WriteItem(
                        index=MetadataIndex(fqn, torch.Size(offsets)),
                        type=WriteItemType.SHARD,
                        tensor_data=TensorWriteData(
                            chunk=ChunkStorageMetadata(offsets=torch.Size(offsets), sizes=torch.Size(sizes)),
                            properties=TensorProperties(dtype=ent.dtype),
                            size=torch.Size(ent.global_shape)),
                    ))
        self.plan = SavePlan(items, plan.storage_data, plan.planner_data)
        return self.plan

    def resolve_data(self, write_item: WriteItem):
        ent = self._entries.get(write_item.index.fqn)
        if ent is None:
            return super().resolve_data(write_item)
        off = tuple(write_item.index.offset)
        for offsets, _sizes, t in ent.chunks:
            if tuple(offsets) == off:
                t = t.detach()
                if t.dtype != ent.dtype:
                    t = t.to(ent.dtype)
                return t
        raise KeyError(f"chunk {off} of {write_item.index.fqn} not found")


class ChunkLoadPlanner(DefaultLoadPlanner):
    def __init__(self, allow_partial_load: bool = False):
        super().__init__(flatten_state_dict=False, allow_partial_load=allow_partial_load)
        self._entries: dict[str, ShardedEntry] = {}
        self._staging: dict[tuple[str, tuple], torch.Tensor] = {}
        self._nested: dict[str, Any] = {}

    def set_up_planner(self, state_dict, metadata=None, is_coordinator=False):
        flat: dict[str, Any] = {}
        _flatten("", state_dict, flat)
        self._nested = state_dict
        self._entries = {k: v for k, v in flat.items() if isinstance(v, ShardedEntry)}
        self._plain = {k: v for k, v in flat.items() if not isinstance(v, ShardedEntry)}
        super().set_up_planner(self._plain, metadata, is_coordinator)

    def create_local_plan(self) -> LoadPlan:
        plan = super().create_local_plan()
        items = list(plan.items)
        for fqn, ent in self._entries.items():
            md = self.metadata.state_dict_metadata.get(fqn)
            if md is None:
                if self.allow_partial_load:
                    continue
                raise RuntimeError(f"missing key in checkpoint: {fqn}")
            if not isinstance(md, TensorStorageMetadata):
                raise RuntimeError(f"checkpoint entry {fqn} is not a tensor")
            if tuple(md.size) != tuple(ent.global_shape):
                raise RuntimeError(f"shape mismatch for {fqn}: checkpoint {tuple(md.size)} vs model {ent.global_shape}")
            local = [ChunkStorageMetadata(offsets=torch.Size(o), sizes=torch.Size(s)) for o, s, _ in ent.chunks]
            items += create_read_items_for_chunk_list(fqn, md, local)
        return LoadPlan(items, plan.storage_data, plan.planner_data)

    def lookup_tensor(self, index: MetadataIndex) -> torch.Tensor:
        ent = self._entries.get(index.fqn)
        if ent is None:
            return super().lookup_tensor(index)
        if index.index is not None and index.index < len(ent.chunks) and (
                index.offset is None or tuple(ent.chunks[index.index][0]) == tuple(index.offset)):
            return ent.chunks[index.index][2]
        for offsets, _sizes, t in ent.chunks:
            if tuple(offsets) == tuple(index.offset):
                return t
        raise KeyError(f"chunk {index.offset} of {index.fqn} not found")

    def finish_plan(self, plan):
        return plan

    def plain_state(self) -> dict[str, Any]:
        # the base planner may have replaced the dict it was given by a processed copy
        return self.state_dict


def _unflatten_into(nested: dict, flat: dict[str, Any], prefix: str = "") -> None:
    for k, v in list(nested.items()):
        key = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, dict):
            _unflatten_into(v, flat, key)
        elif not isinstance(v, ShardedEntry) and key in flat:
            nested[k] = flat[key]


# ----------------------------------------------------------------------
# manager
# ----------------------------------------------------------------------
def _purge_worker(q: "queue.Queue[str | None]") -> None:
    while True:
        path = q.get()
        if path is None:
            return
        try:
            t = time.monotonic()
            fsys.rmtree(path, ignore_errors=True)
            logger.info(f"Checkpointer deleted {path} in {time.monotonic() - t:.2f}s")
        except Exception as e:  # the purge thread must survive failed deletes
            logger.warning(f"failed to delete {path}: {e}")


class CheckpointManager(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        enable: bool = False
        folder: str = "checkpoint"
        interval: int = 500
        initial_load_path: str | None = None
        initial_load_model_only: bool = True
        initial_load_in_hf: bool = False
        initial_load_in_hf_quantized: bool = False
        last_save_model_only: bool = True
        last_save_in_hf: bool = False
        export_dtype: Literal["float16", "bfloat16", "float32"] = "float32"
        async_mode: Literal["disabled", "async", "async_with_pinned_mem"] = "disabled"
        keep_latest_k: int = 10
        load_step: int = -1
        exclude_from_loading: list[str] = field(default_factory=list)
        enable_first_step_checkpoint: bool = False
        create_seed_checkpoint: bool = False
        load_only: bool = False
        storage: Literal["dcp", "torch_save"] = "dcp"
        """``dcp``: torch.distributed.checkpoint files; ``torch_save``: one ``torch.save`` file per rank with global chunk
        offsets (``TorchCheckpointingManager``); both load across layouts."""

    def __new__(cls, config=None, **kw):
        if cls is CheckpointManager and config is not None and getattr(config, "storage", "dcp") == "torch_save":
            return object.__new__(TorchCheckpointingManager)
        return object.__new__(cls)

    def __init__(self, config: "CheckpointManager.Config", *, trainer=None, dump_folder: str = "./outputs",
                 pdims=None, **_):
        self.config = config
        self.trainer = trainer
        self.pdims = pdims
        self.enable = config.enable
        # an fsspec URI as checkpoint.folder (s3://..., gs://..., memory://...) is used as it is
        self.folder = config.folder if fsys.is_remote(config.folder) else fsys.join(dump_folder, config.folder)
        self.async_mode = AsyncMode(config.async_mode)
        self._bg: threading.Thread | None = None
        self._bg_error: BaseException | None = None
        self._stage_event = None
        self._gloo = None
        self._purge_q: queue.Queue | None = None
        self._purge_t: threading.Thread | None = None
        if not self.enable:
            return
        c = config
        if c.last_save_in_hf and not c.last_save_model_only:
            raise ValueError("checkpoint.last_save_in_hf requires last_save_model_only")
        if c.initial_load_in_hf_quantized and not c.initial_load_in_hf:
            raise ValueError("initial_load_in_hf_quantized requires initial_load_in_hf")
        if c.keep_latest_k == 1:
            raise ValueError("keep_latest_k=1 would delete the checkpoint being written; use 0 or >= 2")
        if self.async_mode != AsyncMode.DISABLED and dist.is_initialized() and dist.get_world_size() > 1:
            self._gloo = dist.new_group(backend="gloo")
        if c.keep_latest_k > 0:
            self._purge_q = queue.Queue()
            self._purge_t = threading.Thread(target=_purge_worker, args=(self._purge_q,), daemon=True)
            self._purge_t.start()
        logger.info(f"Checkpointing active. Checkpoints will be loaded from and saved to {self.folder}")

    # -- state assembly --------------------------------------------------------
    def _engines(self):
        return self.trainer.engines

    def _model_state(self, dtype=None) -> dict[str, ShardedEntry]:
        out: dict[str, ShardedEntry] = {}
        for e in self._engines():
            out.update(engine_model_state(e, dtype))
        return out

    def _full_state(self) -> dict[str, Any]:
        t = self.trainer
        sd: dict[str, Any] = dict(self._model_state())
        sd[OPTIMIZER] = t.optimizers.state_dict()
        sd[LR_SCHEDULER] = t.lr_schedulers.state_dict()
        sd[DATALOADER] = t.dataloader.state_dict()
        sd[TRAIN_STATE] = t.state_dict()
        return sd

    def _apply_plain(self, sd: dict[str, Any]) -> None:
        t = self.trainer
        if OPTIMIZER in sd:
            t.optimizers.load_state_dict(sd[OPTIMIZER])
        if LR_SCHEDULER in sd:
            t.lr_schedulers.load_state_dict(sd[LR_SCHEDULER])
        if DATALOADER in sd:
            t.dataloader.load_state_dict(sd[DATALOADER])
        if TRAIN_STATE in sd:
            t.load_state_dict(sd[TRAIN_STATE])

    # -- paths -----------------------------------------------------------------
    def _step_dir(self, step: int) -> str:
        return fsys.join(self.folder, f"step-{step}")

    def _find_steps(self, folder: str | None = None) -> list[int]:
        folder = folder or self.folder
        steps = []
        for name in fsys.listdir(folder):
            m = re.fullmatch(r"step-(\d+)", name)
            if not m:
                continue
            inside = fsys.listdir(fsys.join(folder, name))
            if ".metadata" in inside or "model.safetensors.index.json" in inside or any(
                    f.endswith(".safetensors") for f in inside):
                steps.append(int(m.group(1)))
        return sorted(steps)

    def _should_save(self, step: int, last_step: bool) -> bool:
        if not self.enable or self.config.load_only:
            return False
        if step == 1 and self.config.enable_first_step_checkpoint:
            return True
        return last_step or step % self.config.interval == 0

    # -- save ------------------------------------------------------------------
    def save(self, step: int, last_step: bool = False) -> None:
        if not self._should_save(step, last_step):
            return
        sl.add_step_tag("checkpoint_save")
        with sl.span("checkpoint_save"):
            t0 = time.monotonic()
            self.maybe_wait_for_saving()
            path = self._step_dir(step)
            logger.info(f"Saving the checkpoint (or staging if async is enabled) at step {step}")
            if last_step and self.config.last_save_model_only:
                self._save_last_step(step, path)
            elif self.async_mode == AsyncMode.DISABLED:
                self._dcp_save(self._full_state(), path)
            else:
                self._async_save(self._full_state(), path)
            self._purge_stale()
            logger.info(f"Finished saving the checkpoint (or staging) at step {step} in {time.monotonic() - t0:.2f}s")

    def _dcp_save(self, state: dict[str, Any], path: str, group=None) -> None:
        writer_filter = True
        if self.pdims is not None and self.pdims.dp_replicate > 1:
            writer_filter = self.pdims.coords()["dp_replicate"] == 0
        dcp.save(state, checkpoint_id=path, planner=ChunkSavePlanner(writer_rank_filter=writer_filter),
                 process_group=group)

    def _engine_load(self, state: dict[str, Any], path: str) -> None:
        """Fill the tensors of ``state`` (this rank's chunks) and its plain entries from the files under ``path``."""
        planner = ChunkLoadPlanner()
        dcp.load(state, checkpoint_id=path, planner=planner)
        _unflatten_into(state, planner.plain_state())

    def _save_last_step(self, step: int, path: str) -> None:
        c = self.config
        dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[c.export_dtype]
        state = self._model_state(dtype)
        if c.last_save_in_hf:
            self._save_hf(state, path)
        else:
            self._dcp_save(state, path)

    def _stage_to_host(self, state: dict[str, Any]) -> dict[str, Any]:
        """Copy every chunk to pinned host memory on a side stream."""
        pin = self.async_mode == AsyncMode.ASYNC_WITH_PINNED_MEM and torch.cuda.is_available()
        dev = self.trainer.device
        stream = torch.cuda.Stream(dev) if dev.type == "cuda" else None

        def conv(obj):
            if isinstance(obj, ShardedEntry):
                chunks = []
                for o, s, t in obj.chunks:
                    h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
                    h.copy_(t, non_blocking=True)
                    chunks.append((o, s, h))
                return ShardedEntry(obj.global_shape, obj.dtype, chunks)
            if isinstance(obj, dict):
                return {k: conv(v) for k, v in obj.items()}
            if isinstance(obj, torch.Tensor):
                return obj.detach().to("cpu", non_blocking=True)
            return obj

        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(stream):
                staged = conv(state)
                self._stage_event = torch.cuda.Event()
                self._stage_event.record(stream)
        else:
            staged = conv(state)
        return staged

    def _async_save(self, state: dict[str, Any], path: str) -> None:
        staged = self._stage_to_host(state)
        ev = self._stage_event

        def run():
            try:
                if ev is not None:
                    ev.synchronize()
                self._dcp_save(staged, path, group=self._gloo)
            except BaseException as e:
                self._bg_error = e

        self._bg = threading.Thread(target=run, daemon=True)
        self._bg.start()

    def maybe_wait_for_staging(self) -> None:
        """The optimizer must not overwrite tensors that are still being copied to the host."""
        if self._stage_event is not None:
            self._stage_event.synchronize()
            self._stage_event = None

    def maybe_wait_for_saving(self) -> None:
        if self._bg is not None:
            self._bg.join()
            self._bg = None
            if self._bg_error is not None:
                err, self._bg_error = self._bg_error, None
                raise RuntimeError("asynchronous checkpoint save failed") from err

    def _purge_stale(self) -> None:
        k = self.config.keep_latest_k
        if k <= 0 or self._purge_q is None:
            return
        rank = dist.get_rank() if dist.is_initialized() else 0
        if rank != 0:
            return
        steps = self._find_steps()
        for s in steps[:-k] if len(steps) > k else []:
            self._purge_q.put(self._step_dir(s))

    # -- Hugging Face safetensors ------------------------------------------------
    def _gather_full(self, state: dict[str, ShardedEntry]) -> dict[str, torch.Tensor]:
        """Assemble full tensors on rank 0 (model-only export; sizes are modest per tensor)."""
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        names = sorted(state)
        if world > 1:
            all_names: list = [None] * world
            dist.all_gather_object(all_names, names)
            names = sorted(set().union(*map(set, all_names)))
        full: dict[str, torch.Tensor] = {}
        for name in names:
            ent = state.get(name)
            payload = None
            if ent is not None:
                payload = (ent.global_shape, ent.dtype, [(o, s, t.detach().to("cpu", ent.dtype)) for o, s, t in ent.chunks])
            gathered = [payload]
            if world > 1:
                gathered = [None] * world if rank == 0 else None
                dist.gather_object(payload, gathered, dst=0)
            if rank == 0:
                shape = dt = None
                for p in gathered:
                    if p is not None:
                        shape, dt = p[0], p[1]
                out = torch.empty(shape, dtype=dt)
                for p in gathered:
                    if p is None:
                        continue
                    for o, s, t in p[2]:
                        view = out
                        for d, (oo, ss) in enumerate(zip(o, s)):
                            view = view.narrow(d, oo, ss)
                        view.copy_(t.reshape(view.shape))
                full[name] = out
        return full

    def _save_hf(self, state: dict[str, ShardedEntry], path: str) -> None:
        from safetensors.torch import save_file

        spec = self.trainer.model_spec
        if spec.state_dict_adapter is None:
            raise ValueError(f"model {spec.name} has no Hugging Face state-dict adapter")
        full = self._gather_full(state)
        rank = dist.get_rank() if dist.is_initialized() else 0
        if rank == 0:
            adapter = spec.state_dict_adapter(self.trainer.model_config, self.trainer.config.hf_assets_path)
            hf = {k: v.contiguous() for k, v in adapter.to_hf(full).items()}
            os.makedirs(path, exist_ok=True)
            save_file(hf, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
            import json

            index = {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in hf.values())},
                     "weight_map": {k: "model.safetensors" for k in hf}}
            with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
                json.dump(index, f, indent=2)
        if dist.is_initialized():
            dist.barrier()

    def _load_hf(self, path: str, state: dict[str, ShardedEntry]) -> None:
        from safetensors import safe_open

        spec = self.trainer.model_spec
        adapter = spec.state_dict_adapter(self.trainer.model_config, path)
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        # which HF keys are needed, by translating an empty native dict
        native_keys = {k: torch.empty(0) for k in state}
        try:
            wanted = set(adapter.to_hf(native_keys).keys())
        except Exception:
            wanted = None
        hf: dict[str, torch.Tensor] = {}
        for fn in files:
            with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
                for k in f.keys():
                    if wanted is None or k in wanted:
                        hf[k] = f.get_tensor(k)
        native = adapter.from_hf(hf)
        for name, ent in state.items():
            if name not in native:
                raise RuntimeError(f"Hugging Face checkpoint at {path} lacks '{name}'")
            src = native[name]
            if tuple(src.shape) != tuple(ent.global_shape):
                raise RuntimeError(f"shape mismatch for {name}: {tuple(src.shape)} vs {ent.global_shape}")
            for o, s, t in ent.chunks:
                view = src
                for d, (oo, ss) in enumerate(zip(o, s)):
                    view = view.narrow(d, oo, ss)
                t.copy_(view.reshape(t.shape))

    # -- load ------------------------------------------------------------------
    def load(self, step: int = -1) -> bool:
        if not self.enable:
            return False
        c = self.config
        steps = self._find_steps()
        model_only = False
        in_hf = False
        if steps:
            # a checkpoint in the job's own folder always wins: an auto-restarted job resumes
            if step == -1:
                step = steps[-1]
            elif step not in steps:
                raise FileNotFoundError(f"checkpoint.load_step={step} not found in {self.folder} (have {steps})")
            path = self._step_dir(step)
            model_only = step == 0
            in_hf = not fsys.exists(fsys.join(path, ".metadata"))
        elif c.initial_load_path:
            path = c.initial_load_path
            if not fsys.isdir(path):
                raise FileNotFoundError(f"checkpoint.initial_load_path is invalid: {path}")
            model_only = c.initial_load_model_only
            in_hf = c.initial_load_in_hf
            sub = self._find_steps(path)
            if sub and not fsys.exists(fsys.join(path, ".metadata")) and not in_hf:
                path = fsys.join(path, f"step-{sub[-1]}")
        elif c.initial_load_in_hf:
            path = self.trainer.config.hf_assets_path
            model_only = True
            in_hf = True
        else:
            return False
        logger.info(f"Loading the checkpoint from {path}")
        t0 = time.monotonic()
        with sl.span("checkpoint_load"):
            if model_only:
                state: dict[str, Any] = dict(self._model_state())
            else:
                state = self._full_state()
            for key in c.exclude_from_loading:
                if key == MODEL:
                    for k in [k for k, v in state.items() if isinstance(v, ShardedEntry)]:
                        state.pop(k)
                elif key in state:
                    state.pop(key)
                else:
                    raise ValueError(f"checkpoint.exclude_from_loading: unknown key '{key}'")
            if in_hf:
                self._load_hf(path, {k: v for k, v in state.items() if isinstance(v, ShardedEntry)})
            else:
                self._engine_load(state, path)
                self._apply_plain(state)
            for e in self._engines():
                e.publish_params()
        logger.info(f"Finished loading the checkpoint in {time.monotonic() - t0:.2f}s")
        return True

    def create_seed_checkpoint(self) -> None:
        """Model-only checkpoint at step 0 from the freshly initialised weights."""
        path = self._step_dir(0)
        self._dcp_save(dict(self._model_state()), path)
        logger.info(f"Created seed checkpoint at {path}")

    def close(self) -> None:
        if not self.enable:
            return
        self.maybe_wait_for_saving()
        if self._purge_q is not None:
            self._purge_q.put(None)
            self._purge_t.join(timeout=60)


def _box_overlap(off_a, size_a, off_b, size_b):
    """Intersection of two axis-aligned boxes: ``(offset, size)`` or None."""
    lo = tuple(max(a, b) for a, b in zip(off_a, off_b))
    hi = tuple(min(a + x, b + y) for a, x, b, y in zip(off_a, size_a, off_b, size_b))
    if any(h <= l for l, h in zip(lo, hi)):
        return None
    return lo, tuple(h - l for l, h in zip(lo, hi))


class TorchCheckpointingManager(CheckpointManager):
    """Same policy surface (intervals, retention, async modes, model-only export, resume rules) on plain
    ``torch.save`` files instead of DCP: every writer rank stores its chunks (with their global offsets) and its
    plain entries in ``rank-<r>.pt``, rank 0 adds ``.metadata`` with the rank count.  Loading reads the chunk index
    of every rank file (memory-mapped) and copies the overlaps into this rank's chunks, so a checkpoint written with one
    layout loads with another; no collective is used, writers only need a shared folder.  Parity: the interface of
    torchtitan/components/checkpointer/torch_checkpointing.py:121-222 (whose ``_save`` / ``_load`` are not implemented
    there)."""

    Config = CheckpointManager.Config
    _META = ".metadata"

    def _dcp_save(self, state: dict[str, Any], path: str, group=None) -> None:
        import json

        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        writer = not (self.pdims is not None and self.pdims.dp_replicate > 1 and self.pdims.coords()["dp_replicate"] != 0)
        flat: dict[str, Any] = {}
        _flatten("", state, flat)
        payload = {"chunks": {}, "plain": {}}
        for k, v in flat.items():
            if isinstance(v, ShardedEntry):
                if writer:
                    payload["chunks"][k] = {"global_shape": tuple(v.global_shape), "dtype": v.dtype,
                                            "pieces": [(tuple(o), tuple(z), t.detach().to(v.dtype).cpu().clone())
                                                       for o, z, t in v.chunks]}
            else:
                payload["plain"][k] = v.detach().cpu() if isinstance(v, torch.Tensor) else v
        os.makedirs(path, exist_ok=True)
        tmp = os.path.join(path, f"rank-{rank}.pt.tmp")
        torch.save(payload, tmp)
        os.replace(tmp, os.path.join(path, f"rank-{rank}.pt"))
        if dist.is_initialized() and world > 1:
            dist.barrier(group=group)
        if rank == 0:      # written last: a folder without it is an unfinished checkpoint
            with open(os.path.join(path, self._META), "w") as f:
                json.dump({"engine": "torch_save", "ranks": world}, f)
        if dist.is_initialized() and world > 1:
            dist.barrier(group=group)

    def _engine_load(self, state: dict[str, Any], path: str) -> None:
        import json

        with open(os.path.join(path, self._META)) as f:
            meta = json.load(f)
        if meta.get("engine") != "torch_save":
            raise ValueError(f"{path} was not written by the torch.save checkpoint engine")
        flat: dict[str, Any] = {}
        _flatten("", state, flat)
        wanted = {k: v for k, v in flat.items() if isinstance(v, ShardedEntry)}
        covered = {k: [0] * len(v.chunks) for k, v in wanted.items()}
        plain: dict[str, Any] = {}
        for r in range(int(meta["ranks"])):
            data = torch.load(os.path.join(path, f"rank-{r}.pt"), map_location="cpu", mmap=True, weights_only=False)
            for k, v in data["plain"].items():
                plain.setdefault(k, v)
            for k, ent in wanted.items():
                saved = data["chunks"].get(k)
                if saved is None:
                    continue
                if tuple(saved["global_shape"]) != tuple(ent.global_shape):
                    raise ValueError(f"{k}: saved with global shape {saved['global_shape']}, the model has {ent.global_shape}")
                for i, (off, size, dst) in enumerate(ent.chunks):
                    for s_off, s_size, src in saved["pieces"]:
                        box = _box_overlap(off, size, s_off, s_size)
                        if box is None:
                            continue
                        lo, ext = box
                        d = dst.view(size) if dst.dim() != len(size) else dst
                        sl_d = tuple(slice(a - b, a - b + n) for a, b, n in zip(lo, off, ext))
                        sl_s = tuple(slice(a - b, a - b + n) for a, b, n in zip(lo, s_off, ext))
                        with torch.no_grad():
                            d[sl_d].copy_(src.view(s_size)[sl_s].to(d.dtype))
                        n = 1
                        for e in ext:
                            n *= e
                        covered[k][i] += n
        for k, ent in wanted.items():
            for i, (_off, size, _t) in enumerate(ent.chunks):
                n = 1
                for e in size:
                    n *= e
                if covered[k][i] < n:
                    raise KeyError(f"the checkpoint at {path} does not cover '{k}' (chunk {i}: {covered[k][i]} of {n} elements)")
        _unflatten_into(state, {k: v for k, v in plain.items() if k in flat and k not in wanted})


