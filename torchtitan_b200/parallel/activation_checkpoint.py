"""Activation recomputation policies.

* ``selective`` (default, "op" option): GEMM and attention outputs are kept; the
  bandwidth-bound producers (RMSNorm output, SwiGLU activation) are recomputed
  inside the fused autograd functions of :mod:`torchtitan_b200.ops.functional`.
  A numeric ``selective_ac_option`` N instead recomputes every N-th block fully.
  ``selective_ac_option = "op_half_mm"`` is the per-op save list of the reference: every block is recomputed in
  backward except the ops whose outputs are kept from the first forward: attention, and every second GEMM
  (GEMMs whose weight shape matches a module named in ``force_recompute_mm_shapes_by_fqns``, by default the MoE
  router gate, are always recomputed and do not count).  Less memory than "op", one forward GEMM in two run twice.
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

__all__ = ["apply_activation_checkpointing", "checkpoint_block", "half_mm_policy", "forced_recompute_shapes"]


class _SacContext:
    """Makes a per-op checkpoint session current for the first forward (recording) or the recompute (replaying)."""

    def __init__(self, session: "OF.SacSession", replaying: bool):
        self.session, self.replaying = session, replaying

    def __enter__(self):
        self.prev = OF.settings.sac
        self.session.begin(self.replaying)
        OF.settings.sac = self.session
        return self

    def __exit__(self, *exc):
        OF.settings.sac = self.prev
        return False


def half_mm_policy(forced_shapes: set[tuple[int, int]]):
    """Keep attention outputs and the 1st, 3rd, ... GEMM output of a block; GEMMs with a forced shape
    ``(in_features, out_features)`` are always recomputed and are not counted."""

    def policy(kind, shape, session) -> bool:
        if kind == "attention":
            return True
        if kind == "mm":
            if tuple(shape) in forced_shapes:
                return False
            session.mm_count += 1
            return session.mm_count % 2 == 1
        return False

    return policy


def forced_recompute_shapes(block: nn.Module, fqns: list[str]) -> set[tuple[int, int]]:
    """``(in_features, out_features)`` of every linear-like module of ``block`` whose name contains one of ``fqns``."""
    out = set()
    for name, m in block.named_modules():
        w = getattr(m, "weight", None)
        if w is not None and w.dim() == 2 and any(f in name for f in fqns):
            out.add((int(w.shape[1]), int(w.shape[0])))
    return out


def checkpoint_block(block: nn.Module, preserve_rng_state: bool = True, determinism_check: str = "default",
                     debug: bool = False, sac_policy=None) -> None:
    """Wrap ``block.forward`` so the block is recomputed during backward; with ``sac_policy`` the ops it selects
    keep their first-forward outputs (:class:`torchtitan_b200.ops.functional.SacSession`)."""
    if getattr(block, "_ac_wrapped", False):
        return
    inner = block.forward
    extra = {}
    if sac_policy is not None:
        def context_fn():
            session = OF.SacSession(sac_policy)
            block._last_sac_session = session
            return _SacContext(session, False), _SacContext(session, True)

        extra["context_fn"] = context_fn

    @functools.wraps(inner)
    def forward(*args, **kwargs):
        return checkpoint(inner, *args, use_reentrant=False, preserve_rng_state=preserve_rng_state,
                          determinism_check=determinism_check, debug=debug, **extra, **kwargs)

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
        elif opt == "op_half_mm":
            for b in blocks:
                forced = forced_recompute_shapes(b, list(ac.force_recompute_mm_shapes_by_fqns))
                checkpoint_block(b, sac_policy=half_mm_policy(forced), **kw)
        elif opt != "op":
            raise ValueError(f"unknown selective_ac_option '{opt}' ('op', 'op_half_mm' or a positive integer)")
    elif mode == "memory_budget":
        n_full = int(round(len(blocks) * (1.0 - ac.memory_budget)))
        for b in blocks[len(blocks) - n_full:]:
            checkpoint_block(b, **kw)
    else:
        raise ValueError(f"unknown activation checkpoint mode '{mode}'")
