"""Activation recomputation policies.

* ``selective`` (default, "op" option): GEMM and attention outputs are kept; the
  bandwidth-bound producers (RMSNorm output, SwiGLU activation) are recomputed
  inside the fused autograd functions of :mod:`torchtitan_b200.ops.functional`.
  A numeric ``selective_ac_option`` N instead recomputes every N-th block fully.
* ``full``: every block is recomputed in backward (``torch.utils.checkpoint``,
  non-reentrant, RNG state preserved).
* ``none``: all intermediates are kept.
* ``memory_budget``: blocks are fully recomputed from the last one backwards until
  the fraction ``1 - memory_budget`` of blocks is covered (a static stand-in for
  the compiler partitioner the reference relies on).

Parity: torchtitan/distributed/activation_checkpoint.py:112-337.
"""

from __future__ import annotations

import functools

import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from torchtitan_b200.ops import functional as OF

__all__ = ["apply_activation_checkpointing", "checkpoint_block"]


def checkpoint_block(block: nn.Module, preserve_rng_state: bool = True, determinism_check: str = "default",
                     debug: bool = False) -> None:
    """Wrap ``block.forward`` so the block is recomputed during backward."""
    if getattr(block, "_ac_wrapped", False):
        return
    inner = block.forward

    @functools.wraps(inner)
    def forward(*args, **kwargs):
        return checkpoint(inner, *args, use_reentrant=False, preserve_rng_state=preserve_rng_state,
                          determinism_check=determinism_check, debug=debug, **kwargs)

    block.forward = forward
    block._ac_wrapped = True


def apply_activation_checkpointing(model: nn.Module, ac) -> None:
    mode = ac.mode
    OF.settings.recompute = mode != "none"
    blocks = list(model.layers.values())
    kw = dict(preserve_rng_state=ac.preserve_rng_state, determinism_check=ac.determinism_check, debug=ac.debug)
    if mode in ("none",):
        return
    if mode == "full":
        for b in blocks:
            checkpoint_block(b, **kw)
    elif mode == "selective":
        opt = str(ac.selective_ac_option)
        if opt.isdigit():
            every = int(opt)
            if every <= 0:
                raise ValueError("selective_ac_option must be 'op' or a positive integer")
            for i, b in enumerate(blocks):
                if (i + 1) % every == 0:
                    checkpoint_block(b, **kw)
        elif opt != "op":
            raise ValueError(f"unknown selective_ac_option '{opt}'")
    elif mode == "memory_budget":
        n_full = int(round(len(blocks) * (1.0 - ac.memory_budget)))
        for b in blocks[len(blocks) - n_full:]:
            checkpoint_block(b, **kw)
    else:
        raise ValueError(f"unknown activation checkpoint mode '{mode}'")
