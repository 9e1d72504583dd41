"""Policy-gradient losses on folded token streams.

``token_logprobs(logits[T, V], tokens[T])`` -> ``(logp[T], entropy[T])`` in fp32.
``grpo_loss``: clipped importance-weighted surrogate with an optional k3 KL penalty to a reference
policy, averaged over response tokens (GRPO, Shao et al. 2024).  ``dapo_loss``: decoupled clip
range (``eps_low``, ``eps_high``), token-level normalisation, no KL term (DAPO, Yu et al. 2025).
Parity: torchtitan/components/loss.py:318-380 (compute_logprobs) and the experiment's loss module.
"""

from __future__ import annotations

import torch

__all__ = ["token_logprobs", "group_advantages", "grpo_loss", "dapo_loss", "PolicyLoss"]


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


class PolicyLoss:
    """Per-token clipped surrogate on a packed microbatch, normalised by the step's *global* number of valid
    response tokens (so that microbatches and data-parallel ranks simply add up).  ``clip_low == clip_high`` is
    GRPO's clip, a larger ``clip_high`` DAPO's "clip-higher".  Tokens whose generator log-probability is not finite
    are left out rather than trained as if on-policy; the log-ratio is clamped to +-``max_log_ratio`` before the
    exponential.  Returns ``(loss, metrics)``; the metrics are already divided by the global count, so they are
    summed over microbatches and ranks.

    Parity: torchtitan/experiments/rl/losses/grpo.py:17-36, losses/dapo.py:23-136."""

    def __init__(self, clip_low: float = 0.2, clip_high: float = 0.2, max_log_ratio: float = 20.0):
        self.clip_low, self.clip_high, self.max_log_ratio = clip_low, clip_high, max_log_ratio

    def __call__(self, logits, labels, global_valid_tokens, *, generator_logprobs, advantages, loss_mask):
        logp, entropy = token_logprobs(logits, labels.clamp_min(0))
        valid = loss_mask & torch.isfinite(generator_logprobs)
        raw = torch.where(valid, logp - generator_logprobs, torch.zeros_like(logp))
        ratio = torch.exp(raw.clamp(-self.max_log_ratio, self.max_log_ratio))
        clipped = ratio.clamp(1 - self.clip_low, 1 + self.clip_high)
        adv = advantages.detach()
        denom = max(float(global_valid_tokens or 1), 1.0)
        loss = (-torch.minimum(ratio * adv, clipped * adv) * valid).sum() / denom
        with torch.no_grad():
            d = raw.detach()
            stats = {
                "loss/mean": loss.detach(),
                "loss/ratio_mean": (ratio * valid).sum() / denom,
                "loss/ratio_clipped_frac": (((ratio - clipped).abs() > 1e-6) & valid).sum() / denom,
                "bit_wise/logprob_diff/mean": d.sum() / denom,
                "bit_wise/ratio_tokens_different/mean": ((d.abs() > 1e-6) & valid).sum() / denom,
                "bit_wise/logprob_diff/max": d.abs().max() if d.numel() else d.new_zeros(()),
                "trainer/entropy/mean": (entropy * valid).sum() / denom,
            }
        return loss, stats
