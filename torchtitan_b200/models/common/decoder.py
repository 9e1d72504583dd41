"""Decoder-only transformer over folded tokens.

``Decoder.forward(tokens[T], positions[T])`` returns final hidden states (the
trainer feeds them to the fused lm_head + cross-entropy) or logits.  Layers live
in a ``ModuleDict`` keyed by their index as a string, so pipeline stages can drop
entries without renaming the survivors.  Any of ``tok_embeddings``, ``norm`` and
``lm_head`` may be ``None`` on a pipeline stage.

Parity: torchtitan/models/common/decoder.py:41-360 (block = pre-norm attention +
pre-norm FFN/MoE with residuals), FLOPs accounting torchtitan/models/utils.py:412-545.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn as nn

from torchtitan_b200.ops import functional as OF

from .attention import AttentionContext, GQAttention, build_attention_context
from .layers import Embedding, FeedForward, Linear, RMSNorm
from .module import Module, ModuleDict

__all__ = ["TransformerBlock", "Decoder"]


class TransformerBlock(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        attention: Any = None  # GQAttention.Config | MLAttention.Config ...
        feed_forward: FeedForward.Config | None = None
        moe: Any = None  # MoE.Config
        attention_norm: RMSNorm.Config = field(default_factory=RMSNorm.Config)
        ffn_norm: RMSNorm.Config = field(default_factory=RMSNorm.Config)
        layer_id: int = 0

    def __init__(self, config: "TransformerBlock.Config", **_):
        super().__init__(config)
        self.layer_id = config.layer_id
        self.attention = config.attention.build()
        self.attention_norm = config.attention_norm.build()
        self.ffn_norm = config.ffn_norm.build()
        self.feed_forward = config.feed_forward.build() if config.feed_forward is not None else None
        self.moe = config.moe.build() if config.moe is not None else None
        if (self.feed_forward is None) == (self.moe is None):
            raise ValueError("a block needs exactly one of feed_forward / moe")
        # Tensor parallelism without sequence parallelism: the block norms act on the replicated residual stream,
        # before the activation enters a parallel region, so every rank already holds their complete gradient
        # (with sequence parallelism each rank holds the part of its sequence shard and the parts are summed).
        for norm in (self.attention_norm, self.ffn_norm):
            for p in norm.parameters():
                p._tp_grad_complete_without_sp = True

    def forward(self, x: torch.Tensor, positions: torch.Tensor, ctx: AttentionContext | None = None) -> torch.Tensor:
        h = x + self.attention(x, positions, ctx, norm=self.attention_norm)
        if self.feed_forward is not None:
            return h + self.feed_forward(h, norm=self.ffn_norm)
        return h + self.moe(self.ffn_norm(h))


class Decoder(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        vocab_size: int = 0
        n_layers: int = 0
        layers: list = field(default_factory=list)  # list[TransformerBlock.Config]
        tok_embeddings: Embedding.Config = field(default_factory=Embedding.Config)
        norm: RMSNorm.Config = field(default_factory=RMSNorm.Config)
        lm_head: Linear.Config = field(default_factory=Linear.Config)
        enable_weight_tying: bool = False
        max_context_length: int = 2048
        single_document: bool = False
        """Skip document masking (every batch row is one document starting at 0)."""
        final_logit_softcap: float | None = None
        final_logit_multiplier: float = 1.0
        trainable_param_pattern: str | None = None
        """Regular expression of the parameter names that stay trainable (set by the LoRA converter);
        every other parameter is frozen after construction."""

        # -- accounting ---------------------------------------------------
        def update_from_config(self, *, trainer_config=None, **_) -> None:
            if trainer_config is not None:
                ctx = trainer_config.training.max_context_length
                self.max_context_length = ctx
                for blk in self.layers:
                    rope = getattr(blk.attention, "rope", None)
                    if rope is not None:
                        rope.max_context_length = ctx

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int) -> tuple[int, float]:
            from torchtitan_b200.models.utils import count_params_and_flops

            return count_params_and_flops(self, model, seq_len)

    def __init__(self, config: "Decoder.Config", **_):
        super().__init__(config)
        c = config
        c.tok_embeddings.num_embeddings, c.tok_embeddings.embedding_dim = c.vocab_size, c.dim
        c.norm.dim = c.dim
        c.lm_head.in_features, c.lm_head.out_features = c.dim, c.vocab_size
        self.tok_embeddings = c.tok_embeddings.build()
        self.layers = ModuleDict({str(i): blk.build() for i, blk in enumerate(c.layers)})
        self.norm = c.norm.build()
        for p in self.norm.parameters():
            p._tp_grad_complete_without_sp = True     # as for the block norms
        self.lm_head = c.lm_head.build()
        if c.enable_weight_tying:
            self.lm_head.weight = self.tok_embeddings.weight
        self.single_document = c.single_document
        self.cp = None  # set by parallelize when context parallel is on
        self.tp = None
        if c.trainable_param_pattern:
            import re

            pat = re.compile(c.trainable_param_pattern)
            for n, p in self.named_parameters():
                if not pat.search(n):
                    p.requires_grad_(False)

    def build_context(self, positions: torch.Tensor, q_pos: torch.Tensor | None = None) -> AttentionContext:
        return build_attention_context(positions, assume_single_document=self.single_document, cp=self.cp, q_pos=q_pos)

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor | None = None,
                ctx: AttentionContext | None = None, *, return_hidden: bool = False) -> torch.Tensor:
        """``tokens`` are token ids on the first stage, hidden states ``[T, dim]`` otherwise."""
        if positions is None:
            positions = torch.arange(tokens.shape[0], device=tokens.device)
        if ctx is None:
            ctx = self.build_context(positions)
        h = self.tok_embeddings(tokens) if self.tok_embeddings is not None else tokens
        for layer in self.layers.values():
            h = layer(h, positions, ctx)
        if self.norm is not None:
            h = self.norm(h)
        if return_hidden or self.lm_head is None:
            return h
        if self.tp is not None and self.tp.sequence_parallel:
            from torchtitan_b200.parallel import tp_ops

            h = tp_ops.all_gather_rows(h, self.tp)
        return self.output_logits(h)

    def output_logits(self, h: torch.Tensor) -> torch.Tensor:
        """Output projection (with its multiplier and soft cap) of final-norm hidden states, e.g. of the rows a
        generator samples from after ``forward(..., return_hidden=True)``."""
        logits = self.lm_head(h)
        if self.config.final_logit_multiplier != 1.0:
            logits = logits * self.config.final_logit_multiplier
        cap = self.config.final_logit_softcap
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits
