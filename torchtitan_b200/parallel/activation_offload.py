"""Activation offload: tensors saved for backward move to pinned host memory during the forward and
come back just before their backward needs them.

``with offload_activations(min_bytes=...)`` installs saved-tensor hooks.  In the forward, every saved
CUDA tensor of at least ``min_bytes`` (parameters and views of the flat parameter buffers are left
alone) is copied to a pinned host buffer on a side stream that waits for the producing kernel; the
device copy is released as soon as that copy has finished (its memory is handed back to the caching
allocator with ``record_stream``).  In the backward the tensor is copied back on the side stream and
the consuming stream waits for it.  The side stream keeps the PCIe / C2C copies off the compute
stream, so they overlap with the GEMMs of the neighbouring layers.

With 180 GB of HBM this is for long contexts and large local batches; it composes with selective
recomputation (recomputed tensors are never saved, so they are never offloaded).
Parity: torchtitan/experiments/graph_trainer/cpu_offload.py (activation offload as a graph pass
there; saved-tensor hooks and explicit streams here).
"""

from __future__ import annotations

import contextlib

import torch

__all__ = ["offload_activations", "OffloadStats"]


class OffloadStats:
    def __init__(self) -> None:
        self.tensors = 0
        self.bytes = 0


class _Packed:
    __slots__ = ("host", "event", "device", "dtype", "shape")

    def __init__(self, host, event, device, dtype, shape):
        self.host, self.event, self.device, self.dtype, self.shape = host, event, device, dtype, shape


@contextlib.contextmanager
def offload_activations(min_bytes: int = 1 << 20, stats: OffloadStats | None = None, *, force: bool = False):
    """``force`` offloads CPU tensors through a plain copy as well (exercises the hook logic in tests)."""
    stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def pack(t: torch.Tensor):
        nbytes = t.numel() * t.element_size()
        keep = (not isinstance(t, torch.Tensor) or isinstance(t, torch.nn.Parameter) or nbytes < min_bytes
                or t.requires_grad and t.is_leaf or getattr(t, "_base", None) is not None and isinstance(t._base, torch.nn.Parameter))
        if keep or not (t.is_cuda or force):
            return t
        if stats is not None:
            stats.tensors += 1
            stats.bytes += nbytes
        if not t.is_cuda:
            return _Packed(t.detach().clone(), None, t.device, t.dtype, t.shape)
        src = t.detach()
        host = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
        stream.wait_stream(torch.cuda.current_stream(src.device))
        with torch.cuda.stream(stream):
            host.copy_(src if src.is_contiguous() else src.contiguous(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(stream)
        src.record_stream(stream)        # the allocator may reuse the block once the copy has run
        return _Packed(host, ev, src.device, src.dtype, src.shape)

    def unpack(obj):
        if not isinstance(obj, _Packed):
            return obj
        if obj.event is None:
            return obj.host
        with torch.cuda.stream(stream):
            stream.wait_event(obj.event)
            dev = obj.host.to(obj.device, non_blocking=True)
            back = torch.cuda.Event()
            back.record(stream)
        cur = torch.cuda.current_stream(obj.device)
        cur.wait_event(back)
        dev.record_stream(cur)
        return dev

    with torch.autograd.graph.saved_tensors_hooks(pack, unpack):
        yield stats
