"""CUDA-graph execution of the forward + backward pass.

``CUDAGraphRunner(fn)`` runs ``fn(*tensors)`` eagerly on the first call of a key (allocator and
library warm-up), captures it into a ``torch.cuda.CUDAGraph`` on the second, and from then on
copies the call's tensors into the captured static inputs and replays.  Shapes, dtypes and the
Python control flow of ``fn`` must not change between calls of the same key; the trainer keys
graphs by the microbatch position inside a step (the first microbatch overwrites the gradient
buffers, later ones accumulate, which are different kernels).  Host-side state that ``fn`` mutates
(the sharded engine's "gradients are valid" flags) is re-applied after each replay through
``after_replay``.  Not used with pipeline parallelism or with the NCCL expert-parallel dispatcher,
which synchronises with the host.  Parity: torchtitan/distributed/cudagraph.py:39-410.
"""

from __future__ import annotations

from typing import Callable

import torch

__all__ = ["CUDAGraphRunner"]


class _Captured:
    __slots__ = ("graph", "inputs", "output", "state")


class CUDAGraphRunner:
    def __init__(self, fn: Callable, *, snapshot: Callable | None = None, after_replay: Callable | None = None):
        self.fn = fn
        self.snapshot = snapshot
        self.after_replay = after_replay
        self._seen: dict = {}
        self._graphs: dict = {}
        self._pool = None

    def __call__(self, key, *tensors: torch.Tensor):
        if key in self._graphs:
            c = self._graphs[key]
            for dst, src in zip(c.inputs, tensors):
                dst.copy_(src, non_blocking=True)
            c.graph.replay()
            if self.after_replay is not None:
                self.after_replay(c.state)
            return c.output
        if key not in self._seen:
            self._seen[key] = True
            return self.fn(*tensors)                      # eager warm-up call (a real step)
        c = _Captured()
        c.inputs = [t.clone() for t in tensors]
        c.graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(c.graph, pool=self._pool):
            c.output = self.fn(*c.inputs)
        c.state = self.snapshot() if self.snapshot is not None else None
        self._graphs[key] = c
        c.graph.replay()                                   # capture records, replay executes this call
        return c.output
