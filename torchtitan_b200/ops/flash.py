"""Autograd front-end of the tcgen05 flash-attention kernels (head dimension 128, bf16).

``flash_attention`` takes folded tokens ``q[Tq,Hq,128]``, ``k/v[Tk,Hkv,128]`` (views with a
contiguous last dimension are fine, e.g. slices of a packed QKV projection) and returns
``o[Tq,Hq,128]``; ``flash_attention_lse`` also returns the log-sum-exp ``[Hq,Tq]`` so that
partial results over different key ranges can be merged (context parallelism).

Masks: causal with an offset (row ``i`` sees keys ``j <= i + causal_offset``), an optional
``kv_first[Tq]`` (int32, non-decreasing): the first key each query may see, which is how
packed documents are separated, and an optional sliding ``window`` (row ``i`` sees the last
``window`` keys up to ``i + causal_offset``).  ``sinks[Hq]`` adds one learned logit per head to the
softmax denominator (GPT-OSS attention sinks, torchtitan/models/gpt_oss/model.py:34-47); its
gradient is ``-sum_i exp(sink - lse_i) * delta_i``.  The library counterpart in the reference is flex / varlen
attention (torchtitan/models/common/attention.py:109-362).
"""

from __future__ import annotations

import torch

from . import ext

__all__ = ["flash_attention", "flash_attention_lse", "supported"]


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return (
        q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
        and q.dim() == 3 and q.shape[-1] == 128 and k.shape[-1] == 128 and v.shape[-1] == 128
        and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
        and q.shape[1] % k.shape[1] == 0
    )


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, causal_offset, kv_first, packed_grad, window=0, sinks=None):
        ops = ext.require()
        sinks_f = sinks.detach().float().contiguous() if sinks is not None else None
        from .functional import _sac_run

        o, lse = _sac_run("attention", None,
                          lambda: ops.flash_fwd(q, k, v, scale, causal, causal_offset, kv_first, window, sinks_f))
        ctx.save_for_backward(q, k, v, o, lse, kv_first if kv_first is not None else torch.empty(0),
                              sinks_f if sinks_f is not None else torch.empty(0))
        ctx.has_first = kv_first is not None
        ctx.has_sinks = sinks is not None
        ctx.sink_dtype = sinks.dtype if sinks is not None else None
        ctx.args = (scale, causal, causal_offset, window)
        ctx.packed_grad = packed_grad
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _d_lse):
        q, k, v, o, lse, kv_first, sinks_f = ctx.saved_tensors
        scale, causal, causal_offset, window = ctx.args
        ops = ext.require()
        if not d_o.is_contiguous():
            d_o = d_o.contiguous()
        dq = dk = dv = None
        if ctx.packed_grad and _same_packed_storage(q, k, v):
            # q, k, v are adjacent head slices of one [T, H_total, D] projection output: write the three
            # gradients into one tensor of that shape, so autograd adds views instead of concatenating.
            T, hq, hkv = q.shape[0], q.shape[1], k.shape[1]
            packed = torch.empty(T, hq + 2 * hkv, q.shape[2], dtype=q.dtype, device=q.device)
            dq, dk, dv = packed[:, :hq], packed[:, hq:hq + hkv], packed[:, hq + hkv:]
        dq, dk, dv = ops.flash_bwd(d_o, q, k, v, o, lse, scale, causal, causal_offset,
                                   kv_first if ctx.has_first else None, dq, dk, dv, window)
        d_sinks = None
        if ctx.has_sinks and ctx.needs_input_grad[9]:
            delta = (d_o.float() * o.float()).sum(-1)                                   # [Tq, Hq]
            d_sinks = -(torch.exp(sinks_f[None, :] - lse.t()) * delta).sum(0).to(ctx.sink_dtype)
        return dq, dk, dv, None, None, None, None, None, None, d_sinks


def _same_packed_storage(q, k, v) -> bool:
    if not (q.shape[0] == k.shape[0] == v.shape[0] and q.stride() == k.stride() == v.stride()):
        return False
    esz = q.element_size()
    d = q.shape[2]
    return (
        q.stride(1) == d
        and k.data_ptr() == q.data_ptr() + q.shape[1] * d * esz
        and v.data_ptr() == k.data_ptr() + k.shape[1] * d * esz
        and q.stride(0) == (q.shape[1] + 2 * k.shape[1]) * d
    )


def flash_attention_lse(q, k, v, scale: float, *, causal: bool = True, causal_offset: int = 0,
                        kv_first: torch.Tensor | None = None, window: int | None = None,
                        sinks: torch.Tensor | None = None):
    return _FlashFn.apply(q, k, v, float(scale), bool(causal), int(causal_offset), kv_first, True,
                          int(window or 0), sinks)


def flash_attention(q, k, v, scale: float, *, causal: bool = True, causal_offset: int = 0,
                    kv_first: torch.Tensor | None = None, window: int | None = None,
                    sinks: torch.Tensor | None = None) -> torch.Tensor:
    return flash_attention_lse(q, k, v, scale, causal=causal, causal_offset=causal_offset, kv_first=kv_first,
                               window=window, sinks=sinks)[0]


# ---------------------------------------------------------------------------------------------
# Block-level entry points without autograd: one query block against one key block, the pieces
# that context-parallel attention merges.  CUDA tensors of a supported shape run the tcgen05
# kernels, everything else the dense fp32 reference with the same local-index mask semantics.
def _use_kernels(q, k, v) -> bool:
    from . import functional as OF

    return OF.settings.attention == "native" and supported(q, k, v)


def block_fwd(q, k, v, scale: float, *, causal: bool = True, causal_offset: int = 0, kv_first=None, window: int = 0):
    """``(o [Tq, Hq, D], lse [Hq, Tq] fp32)``; rows without a visible key give ``o = 0``, ``lse = -inf``."""
    if _use_kernels(q, k, v):
        from .functional import _count

        _count()
        return ext.require().flash_fwd(q, k, v, float(scale), bool(causal), int(causal_offset), kv_first, int(window), None)
    from . import reference as ref

    return ref.block_attention_fwd(q, k, v, scale, causal, causal_offset, kv_first, window)


def block_bwd(d_o, q, k, v, o, lse, scale: float, *, causal: bool = True, causal_offset: int = 0, kv_first=None,
              window: int = 0):
    """Gradients of one block given the (possibly merged) output ``o`` and ``lse`` of the whole row."""
    if _use_kernels(q, k, v):
        from .functional import _count

        _count(3)
        return ext.require().flash_bwd(d_o.contiguous(), q, k, v, o.contiguous(), lse, float(scale), bool(causal),
                                       int(causal_offset), kv_first, None, None, None, int(window))
    from . import reference as ref

    return ref.block_attention_bwd(d_o, q, k, v, o, lse, scale, causal, causal_offset, kv_first, window)


def merge_(acc_o: torch.Tensor, acc_lse: torch.Tensor, o: torch.Tensor, lse: torch.Tensor) -> None:
    """Fold a block's ``(o, lse)`` into the running fp32 pair ``acc_o [T, H, D]``, ``acc_lse [H, T]`` (in place)."""
    if acc_o.is_cuda and o.dtype == torch.bfloat16 and o.shape[-1] == 128 and ext.available():
        from .functional import _count

        _count()
        ext.require().attn_merge_(acc_o, acc_lse, o.contiguous(), lse)
        return
    from . import reference as ref

    ref.attention_merge_(acc_o, acc_lse, o, lse)
