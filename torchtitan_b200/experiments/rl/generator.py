"""A sampling generator that runs the trainer's own decoder (no separate inference engine): the
weights the policy is trained with are the weights that act, so no weight sync is needed on one
process.  Decoding recomputes the prefix each step (no KV cache), which is adequate for the short
rollouts of tests and small experiments; parity target: the vLLM generator of
torchtitan/experiments/rl, which shares model definitions with the trainer."""

from __future__ import annotations

import torch

from .rollout import Rollout

__all__ = ["SamplingGenerator"]


class SamplingGenerator:
    def __init__(self, model, *, temperature: float = 1.0, top_k: int = 0, eos_id: int | None = None, seed: int = 0):
        self.model = model
        self.temperature = temperature
        self.top_k = top_k
        self.eos_id = eos_id
        self.gen = torch.Generator().manual_seed(seed)
        self.policy_version = 0

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> Rollout:
        dev = next(self.model.parameters()).device
        seq = prompt.to(dev)
        lps = []
        for _ in range(max_new_tokens):
            logits = self.model(seq, torch.arange(seq.numel(), device=dev))[-1].float()
            if self.temperature <= 0:
                nxt = logits.argmax()
                lp = torch.log_softmax(logits, -1)[nxt]
            else:
                logits = logits / self.temperature
                if self.top_k:
                    kth = logits.topk(self.top_k).values[-1]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                probs = torch.softmax(logits, -1)
                nxt = torch.multinomial(probs.cpu(), 1, generator=self.gen)[0].to(dev)
                lp = torch.log(probs[nxt])
            seq = torch.cat([seq, nxt.view(1)])
            lps.append(lp)
            if self.eos_id is not None and int(nxt) == self.eos_id:
                break
        n = len(lps)
        return Rollout(prompt=prompt.cpu(), response=seq[-n:].cpu(), logprobs=torch.stack(lps).cpu(),
                       policy_version=self.policy_version)
