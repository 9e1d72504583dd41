"""Train Hugging Face ``transformers`` causal-LM architectures with this framework's folded-token
interface, loss and data pipeline (parity: torchtitan/experiments/transformers_modeling_backend).

``HFCausalLM(config_or_name)`` builds the architecture from a ``transformers`` config (random
init) and exposes ``forward(tokens[T], positions[T]) -> logits[T, V]``; documents are kept apart by
passing ``position_ids`` that restart per document together with a block-diagonal causal mask.
``hf_train_steps`` is a minimal data-parallel loop (gradient averaging over the world group)."""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ["HFCausalLM", "hf_train_steps"]


class HFCausalLM(nn.Module):
    def __init__(self, config, *, attn_implementation: str = "sdpa", dtype=torch.float32):
        super().__init__()
        from transformers import AutoConfig, AutoModelForCausalLM

        if isinstance(config, str):
            config = AutoConfig.from_pretrained(config)
        config._attn_implementation = attn_implementation
        self.hf = AutoModelForCausalLM.from_config(config).to(dtype)
        self.vocab_size = config.vocab_size

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        T = tokens.shape[0]
        if positions is None:
            positions = torch.arange(T, device=tokens.device)
        doc = torch.cumsum((positions == 0).long(), 0)
        allowed = (doc[:, None] == doc[None, :]) & torch.ones(T, T, dtype=torch.bool, device=tokens.device).tril()
        mask = torch.zeros(T, T, device=tokens.device, dtype=self.hf.dtype).masked_fill(~allowed, torch.finfo(self.hf.dtype).min)
        out = self.hf(input_ids=tokens[None], position_ids=positions[None], attention_mask=mask[None, None])
        return out.logits[0]


def hf_train_steps(model: HFCausalLM, batches, *, lr: float = 3e-4, max_norm: float = 1.0) -> list[float]:
    """``batches``: iterable of ``(tokens[T], positions[T], labels[T])``; returns the per-step losses."""
    opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1)
    losses = []
    for tokens, positions, labels in batches:
        logits = model(tokens, positions)
        loss = nn.functional.cross_entropy(logits.float(), labels, ignore_index=-100)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        if dist.is_initialized() and dist.get_world_size() > 1:
            for p in model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm)
        opt.step()
        losses.append(float(loss.detach()))
    return losses
