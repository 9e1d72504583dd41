"""Policy-gradient losses on folded token streams.

``token_logprobs(logits[T, V], tokens[T])`` -> ``(logp[T], entropy[T])`` in fp32.
``grpo_loss``: clipped importance-weighted surrogate with an optional k3 KL penalty to a reference
policy, averaged over response tokens (GRPO, Shao et al. 2024).  ``dapo_loss``: decoupled clip
range (``eps_low``, ``eps_high``), token-level normalisation, no KL term (DAPO, Yu et al. 2025).
Parity: torchtitan/components/loss.py:318-380 (compute_logprobs) and the experiment's loss module.
"""

from __future__ import annotations

import torch

__all__ = ["token_logprobs", "group_advantages", "grpo_loss", "dapo_loss"]


def token_logprobs(logits: torch.Tensor, tokens: torch.Tensor, *, with_entropy: bool = True):
    lp = torch.log_softmax(logits.float(), dim=-1)
    chosen = lp.gather(-1, tokens.long().unsqueeze(-1)).squeeze(-1)
    if not with_entropy:
        return chosen, None
    return chosen, -(lp.exp() * lp).sum(-1)


def group_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-6) -> torch.Tensor:
    """``rewards[N]`` with ``N = n_prompts * group_size`` -> per-sample advantage, normalised inside each
    prompt's group of responses."""
    r = rewards.float().view(-1, group_size)
    return ((r - r.mean(dim=1, keepdim=True)) / (r.std(dim=1, keepdim=True, unbiased=False) + eps)).reshape(-1)


def _surrogate(logp, old_logp, adv, mask, eps_low, eps_high):
    ratio = torch.exp(logp - old_logp.detach())
    a = adv.detach()
    obj = torch.minimum(ratio * a, ratio.clamp(1 - eps_low, 1 + eps_high) * a)
    return obj * mask


def grpo_loss(logp, old_logp, adv, mask, *, ref_logp=None, clip_eps: float = 0.2, kl_coef: float = 0.0):
    """All arguments are per token ``[T]``; ``mask`` selects response tokens; ``adv`` holds the sample's
    advantage on each of its tokens."""
    mask = mask.float()
    n = mask.sum().clamp_min(1.0)
    loss = -_surrogate(logp, old_logp, adv, mask, clip_eps, clip_eps).sum() / n
    stats = {"ratio_mean": float((torch.exp(logp.detach() - old_logp) * mask).sum() / n)}
    if ref_logp is not None and kl_coef:
        d = ref_logp.detach() - logp
        kl = (torch.exp(d) - d - 1.0) * mask       # k3 estimator: unbiased, non-negative
        loss = loss + kl_coef * kl.sum() / n
        stats["kl"] = float(kl.detach().sum() / n)
    return loss, stats


def dapo_loss(logp, old_logp, adv, mask, *, eps_low: float = 0.2, eps_high: float = 0.28):
    mask = mask.float()
    n = mask.sum().clamp_min(1.0)
    return -_surrogate(logp, old_logp, adv, mask, eps_low, eps_high).sum() / n, {}
