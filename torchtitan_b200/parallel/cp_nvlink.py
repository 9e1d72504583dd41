"""Context-parallel KV exchange over NVLink peer memory instead of NCCL.

Forward (all-gather): every rank copies its K (or V) chunk into a symmetric staging buffer, a
bounded flag barrier makes the chunks visible, and one kernel pulls all peers' chunks with plain
peer loads into a local buffer (``all_gather_pull``): each remote byte crosses NVLink once and the
attention kernel then reads local memory.  Backward (reduce-scatter): the full-sequence gradient
is staged, and each rank sums its own rows from all peers (``reduce_scatter_pull``, fp32 sum).
A second barrier after each pull keeps a fast rank from overwriting a buffer that is still read.

The waits are bounded (status word, no trap); NVLS / multimem is not used.
"""

from __future__ import annotations

import torch

from torchtitan_b200.ops import ext
from torchtitan_b200.ops.functional import _count

from .symm import _GroupArena

__all__ = ["CPNvlink"]


class CPNvlink:
    def __init__(self, group, device: torch.device, nbytes: int = 256 << 20):
        self.arena = _GroupArena(group, device, nbytes)
        self.size, self.rank = self.arena.size, self.arena.rank
        self.capacity = nbytes
        self.stage = self.arena.buf[:nbytes]

    def _ptrs(self) -> list[int]:
        return list(self.arena.base_ptrs)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``x[n, ...]`` of every rank -> ``[size * n, ...]``, rank-major."""
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        if nbytes % 16 or nbytes > self.capacity:
            raise ValueError(f"cp nvlink all-gather: {nbytes} bytes per rank (capacity {self.capacity}, multiple of 16 needed)")
        self.stage[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self.arena.barrier()
        _count()
        ext.require().all_gather_pull(self._ptrs(), self.rank, nbytes, out)
        self.arena.barrier()
        return out

    def reduce_scatter(self, full: torch.Tensor) -> torch.Tensor:
        """``full[size * n, ...]`` (rank-major) of every rank -> the sum of this rank's ``n`` rows."""
        full = full.contiguous()
        if full.dtype not in (torch.bfloat16, torch.float32):
            full = full.float()
        nbytes = full.numel() * full.element_size()
        n = full.shape[0] // self.size
        shard_elems = n * (full.numel() // full.shape[0])
        if shard_elems % 8 or nbytes > self.capacity:
            raise ValueError(f"cp nvlink reduce-scatter: {nbytes} bytes (capacity {self.capacity}), shard of {shard_elems} elements")
        self.stage[:nbytes].view(full.dtype).view(full.shape).copy_(full)
        out = torch.empty(shard_elems, dtype=torch.float32, device=full.device)
        self.arena.barrier()
        _count()
        ext.require().reduce_scatter_pull(self._ptrs(), self.rank, self.rank * shard_elems, out,
                                          full.dtype == torch.bfloat16, False)
        self.arena.barrier()
        return out.view((n,) + tuple(full.shape[1:])).to(full.dtype)

    # -- ring mode: staged K / V, peers copy a rank's block straight out of its symmetric buffer ------------------
    def stage_pair(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Put this rank's K and V where the peers can read them (two halves of the symmetric buffer) and fence."""
        half = self.capacity // 2
        for slot, t in enumerate((k, v)):
            t = t.contiguous()
            nbytes = t.numel() * t.element_size()
            if nbytes > half:
                raise ValueError(f"cp nvlink ring: {nbytes} bytes per tensor exceed half the staging buffer ({half})")
            self.stage[slot * half: slot * half + nbytes].view(t.dtype).view(t.shape).copy_(t)
        self.arena.barrier()

    def peer_pair(self, rank: int, like_k: torch.Tensor, like_v: torch.Tensor):
        """Views of rank ``rank``'s staged K and V (peer memory; read them with copies or plain loads only)."""
        half = self.capacity // 2
        out = []
        for slot, t in enumerate((like_k, like_v)):
            es = t.element_size()
            out.append(self.arena.handle.get_buffer(rank, tuple(t.shape), t.dtype, (slot * half) // es))
        return out

    def release(self) -> None:
        """Every rank has finished reading the staged tensors (before they are staged again)."""
        self.arena.barrier()

    def check_status(self) -> None:
        v = int(self.arena.status.item())
        if v:
            self.arena.status.zero_()
            raise RuntimeError(f"a bounded device wait expired (status {v:#x}) in the context-parallel NVLink exchange")
