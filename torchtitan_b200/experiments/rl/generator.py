"""Generators that run the trainer's own decoder definitions (no separate inference engine; parity target: the
vLLM generator of torchtitan/experiments/rl/generate.py, which shares model definitions with the trainer).

``SamplingGenerator`` recomputes the prefix for every new token (the oracle of the tests);
``CachedGenerator`` prefills once and then decodes one row per step against a key/value cache;
``WeightSync`` pushes the trainer's weights into a generator's copy of the model, in one process or over a
process group, and stamps the policy version that the rollout buffer uses to drop stale samples."""

from __future__ import annotations

import contextlib

import torch

from .rollout import SampledResponse

__all__ = ["SamplingGenerator", "CachedGenerator", "WeightSync", "frozen_router_counters"]


@contextlib.contextmanager
def frozen_router_counters(model):
    """Forward passes inside this block do not count towards the MoE routers' expert-load statistics (they drive
    the trainer's balancing bias, and generated tokens are not training tokens)."""
    saved = [(m, m.tokens_per_expert_E.clone()) for m in model.modules()
             if isinstance(getattr(m, "tokens_per_expert_E", None), torch.Tensor)]
    try:
        yield
    finally:
        for m, t in saved:
            m.tokens_per_expert_E.copy_(t)


class SamplingGenerator:
    def __init__(self, model, *, temperature: float = 1.0, top_k: int = 0, eos_id: int | None = None, seed: int = 0):
        self.model = model
        self.temperature = temperature
        self.top_k = top_k
        self.eos_id = eos_id
        self.gen = torch.Generator().manual_seed(seed)
        self.policy_version = 0

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> SampledResponse:
        dev = next(self.model.parameters()).device
        seq = prompt.to(dev)
        lps = []
        stack = contextlib.ExitStack()
        stack.enter_context(frozen_router_counters(self.model))
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
        stack.close()
        n = len(lps)
        return SampledResponse(prompt=prompt.cpu(), response=seq[-n:].cpu(), logprobs=torch.stack(lps).cpu(),
                       policy_version=self.policy_version)


class CachedGenerator(SamplingGenerator):
    """Incremental decoding with a key/value cache on the training model's own modules: the prompt is
    prefilled in one pass, every further token runs one row through the blocks and attends to the cached keys
    (``models.common.attention.KVCache``).  The generator can hold its own copy of the model (another device
    or process); ``WeightSync`` refreshes it and bumps ``policy_version``."""

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> SampledResponse:
        from torchtitan_b200.models.common.attention import AttentionContext, KVCache

        dev = next(self.model.parameters()).device
        cache = KVCache()
        ctx = AttentionContext(kv_cache=cache)
        seq = prompt.to(dev)
        step_in, pos0 = seq, 0
        out_tokens, lps = [], []
        was_training = self.model.training
        self.model.eval()
        stack = contextlib.ExitStack()
        stack.enter_context(frozen_router_counters(self.model))
        for _ in range(max_new_tokens):
            n = step_in.numel()
            positions = torch.arange(pos0, pos0 + n, device=dev)
            logits = self.model(step_in, positions, ctx)[-1].float()
            pos0 += n
            nxt, lp = self._sample(logits)
            out_tokens.append(nxt)
            lps.append(lp)
            step_in = nxt.view(1)
            if self.eos_id is not None and int(nxt) == self.eos_id:
                break
        stack.close()
        self.model.train(was_training)
        return SampledResponse(prompt=prompt.cpu(), response=torch.stack(out_tokens).cpu(), logprobs=torch.stack(lps).cpu(),
                       policy_version=self.policy_version)

    def _sample(self, logits: torch.Tensor):
        if self.temperature <= 0:
            nxt = logits.argmax()
            return nxt, torch.log_softmax(logits, -1)[nxt]
        logits = logits / self.temperature
        if self.top_k:
            kth = logits.topk(self.top_k).values[-1]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        probs = torch.softmax(logits, -1)
        nxt = torch.multinomial(probs.cpu(), 1, generator=self.gen)[0].to(logits.device)
        return nxt, torch.log(probs[nxt])


class WeightSync:
    """Copies the trainer's current weights into a generator's copy of the model and stamps the policy version.

    In one process the parameters are matched by name.  Across processes (``group`` given) the trainer rank
    ``src`` broadcasts every parameter in name order and the generator ranks receive into their copies, the
    NCCL / gloo counterpart of the reference's trainer -> generator weight push."""

    def __init__(self, group=None, src: int = 0):
        self.group, self.src = group, src
        self.version = 0

    @torch.no_grad()
    def push(self, trainer_model, generator: SamplingGenerator, engine=None) -> int:
        if engine is not None and hasattr(engine, "wait_optimizer"):
            engine.wait_optimizer()
        src_params = dict(trainer_model.named_parameters()) if trainer_model is not None else {}
        for name, p in generator.model.named_parameters():
            if self.group is None:
                p.copy_(src_params[name].to(p.device, p.dtype))
            else:
                import torch.distributed as dist

                buf = src_params[name].detach().to(p.dtype).contiguous() if name in src_params and dist.get_rank() == self.src \
                    else torch.empty_like(p)
                dist.broadcast(buf, src=self.src, group=self.group)
                p.copy_(buf.to(p.device))
        self.version += 1
        generator.policy_version = self.version
        return self.version
