"""Batch-invariant execution: a sample's result does not depend on what else is in the batch, so the
log-probabilities the generator reports and the ones the trainer recomputes agree bit for bit (parity:
torchtitan/experiments/rl/batch_invariance.py:25-60, torchtitan/distributed/utils.py:318-388, which swap in
fixed-order reduction kernels and pin NCCL algorithms).

The hand-written kernels of this package are batch-invariant by construction: the GEMM walks K in one fixed
order per output tile (no split-K, tile shape independent of M), norms and the cross entropy reduce inside one
row, and the NVLink reduce-scatter sums ranks in rank order.  Attention walks the key tiles of a row in order: a
sequence's result does not depend on the other sequences of a packed batch as long as it starts on a multiple of
the 128-token tile (pad prompts accordingly); at other offsets the same products are grouped into different
partial sums.  What is not invariant are the library paths (cuBLAS picks kernels by shape), so this mode makes every
silent library route an error instead."""

from __future__ import annotations

import contextlib

from torchtitan_b200.ops import functional as OF

__all__ = ["enable_batch_invariant_mode", "batch_invariant"]


def enable_batch_invariant_mode(enabled: bool = True) -> None:
    OF.settings.strict_native = bool(enabled)
    if enabled:
        OF.settings.gemm = "tcgen05"
        OF.settings.attention = "native"


@contextlib.contextmanager
def batch_invariant():
    prev = (OF.settings.strict_native, OF.settings.gemm, OF.settings.attention)
    enable_batch_invariant_mode(True)
    try:
        yield
    finally:
        OF.settings.strict_native, OF.settings.gemm, OF.settings.attention = prev
