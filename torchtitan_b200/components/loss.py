"""Loss functions.

All losses are *sum over valid tokens / global_valid_tokens*, where the divisor
is the number of non-ignored labels of the whole optimizer step across the data
parallel mesh, so data-parallel gradient averaging is not needed (parity:
torchtitan/components/loss.py:27-62,254-271).

``LinearCrossEntropyLoss`` is the default for decoders: it owns a reference to the
``lm_head`` weight, receives final hidden states and runs the chunked fused
lm_head + CE (the ``[T, V]`` logits never exist), the counterpart of the reference's
``ChunkedLossWrapper`` (loss.py:501-809).  With tensor parallelism the vocabulary
is sharded and the softmax statistics are all-reduced over the tp group (parity:
``_LossParallelCrossEntropy``, loss.py:65-216).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from torchtitan_b200.config import Configurable
from torchtitan_b200.ops import functional as OF
from torchtitan_b200.ops.reference import IGNORE_INDEX

__all__ = ["IGNORE_INDEX", "BaseLoss", "CrossEntropyLoss", "LinearCrossEntropyLoss", "MSELoss", "compute_logprobs",
           "vocab_parallel_linear_cross_entropy"]


class BaseLoss(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    needs_hidden = False

    def __init__(self, config=None, **_):
        self.config = config

    def __call__(self, pred: torch.Tensor, labels: torch.Tensor, global_valid_tokens: torch.Tensor | float):
        raise NotImplementedError


def _inv(n) -> torch.Tensor:
    if isinstance(n, torch.Tensor):
        return 1.0 / n.to(torch.float32).clamp_min(1.0)
    return torch.tensor(1.0 / max(float(n), 1.0))


class CrossEntropyLoss(BaseLoss):
    """CE on materialised logits ``[T, V]``."""

    @dataclass(kw_only=True, slots=True)
    class Config(BaseLoss.Config):
        global_vocab_size: int | None = None

    def __call__(self, pred, labels, global_valid_tokens):
        inv = _inv(global_valid_tokens).to(pred.device)
        return OF.cross_entropy_sum(pred.reshape(-1, pred.shape[-1]), labels.reshape(-1)) * inv


class LinearCrossEntropyLoss(BaseLoss):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseLoss.Config):
        num_chunks: int = 8

    needs_hidden = True

    def __init__(self, config=None, **_):
        super().__init__(config or LinearCrossEntropyLoss.Config())
        self.lm_head = None
        self.tp = None
        self.softcap = None
        self.multiplier = 1.0

    def set_lm_head(self, lm_head, tp=None, softcap: float | None = None, multiplier: float = 1.0) -> None:
        self.lm_head, self.tp, self.softcap, self.multiplier = lm_head, tp, softcap, multiplier

    def __call__(self, hidden, labels, global_valid_tokens):
        if self.lm_head is None:
            raise RuntimeError("LinearCrossEntropyLoss.set_lm_head was not called")
        inv = _inv(global_valid_tokens).to(hidden.device)
        w = self.lm_head.weight
        if self.tp is not None and self.tp.size > 1:
            if self.tp.sequence_parallel:
                from torchtitan_b200.parallel import tp_ops

                hidden = tp_ops.all_gather_rows(hidden, self.tp)
            else:
                from torchtitan_b200.parallel import tp_ops

                hidden = tp_ops.copy_to_tp(hidden, self.tp)
            return vocab_parallel_linear_cross_entropy(hidden, w, labels, inv, self.tp, self.config.num_chunks)
        if self.softcap or self.multiplier != 1.0:
            logits = OF.linear(hidden, w).float() * self.multiplier
            if self.softcap:
                logits = self.softcap * torch.tanh(logits / self.softcap)
            return OF.cross_entropy_sum(logits, labels.reshape(-1)) * inv
        return OF.linear_cross_entropy(hidden, w, labels, inv, self.config.num_chunks)


class MSELoss(BaseLoss):
    def __call__(self, pred, labels, global_valid_tokens=None):
        return torch.nn.functional.mse_loss(pred.float(), labels.float().detach())


def compute_logprobs(logits: torch.Tensor, tokens: torch.Tensor, with_entropy: bool = False):
    """Per-token log-probabilities (and optionally entropies) in fp32."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    lp = lf.gather(-1, tokens.clamp_min(0).unsqueeze(-1)).squeeze(-1) - lse
    if not with_entropy:
        return lp
    p = torch.softmax(lf, dim=-1)
    ent = lse - (p * lf).sum(dim=-1)
    return lp, ent


class _VocabParallelLinearCE(torch.autograd.Function):
    """Chunked lm_head + CE with the vocabulary sharded over the tp group."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, inv_tokens, tp, num_chunks):
        h2 = hidden.reshape(-1, hidden.shape[-1])
        lab = labels.reshape(-1)
        T = h2.shape[0]
        vloc = weight.shape[0]
        v0 = tp.rank * vloc
        loss = torch.zeros((), dtype=torch.float32, device=h2.device)
        dh = torch.zeros_like(h2)
        mg = getattr(weight, "main_grad", None)
        dw = None if mg is not None else torch.zeros(weight.shape, dtype=torch.float32, device=h2.device)
        chunk = max(1, -(-T // max(1, num_chunks)))
        scale = inv_tokens.to(torch.float32)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            logits = OF.gemm_nt(h2[s:e], weight).float()
            lb = lab[s:e]
            valid = lb != IGNORE_INDEX
            mx = logits.max(dim=-1).values
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=tp.group)
            ex = torch.exp(logits - mx[:, None])
            se = ex.sum(dim=-1)
            dist.all_reduce(se, group=tp.group)
            local = lb - v0
            mine = (local >= 0) & (local < vloc) & valid
            safe = local.clamp(0, vloc - 1)
            tgt = torch.where(mine, logits.gather(-1, safe[:, None]).squeeze(-1), torch.zeros_like(mx))
            dist.all_reduce(tgt, group=tp.group)
            loss += ((torch.log(se) + mx - tgt) * valid).sum()
            p = ex / se[:, None]
            p.scatter_add_(-1, safe[:, None], -mine.to(p.dtype)[:, None])
            p = (p * valid[:, None] * scale).to(h2.dtype)
            dh[s:e] = OF.gemm_nn(p, weight)
            if mg is not None:
                acc = getattr(weight, "_main_grad_written", False)
                OF.gemm_tn(p, h2[s:e], out=mg.view(weight.shape), accumulate=acc)
                weight._main_grad_written = True
            else:
                dw.addmm_(p.t().float(), h2[s:e].float())
        # dh stays a partial sum over the vocabulary shards: the caller's all-gather /
        # copy-to-tp autograd function reduces it in its backward
        ctx.save_for_backward(dh, dw)
        ctx.weight = weight
        ctx.hshape = hidden.shape
        return loss * scale

    @staticmethod
    def backward(ctx, dloss):
        dh, dw = ctx.saved_tensors
        dwr = None
        if dw is not None:
            dwr = (dw * dloss).to(ctx.weight.dtype)
        return (dh * dloss.to(dh.dtype)).view(ctx.hshape), dwr, None, None, None, None


def vocab_parallel_linear_cross_entropy(hidden, weight, labels, inv_tokens, tp, num_chunks=8):
    if hidden.dtype != weight.dtype:
        hidden = hidden.to(weight.dtype)
    return _VocabParallelLinearCE.apply(hidden, weight, labels, inv_tokens, tp, num_chunks)
