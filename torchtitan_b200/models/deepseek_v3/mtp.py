"""Multi-token prediction (DeepSeek-V3): extra decoder depths that predict tokens further ahead.

Depth ``k`` (1-based) fuses the hidden state of depth ``k - 1`` with the embedding of the token
``k`` positions ahead,

    h_k = Block_k( eh_proj( cat( enorm(emb(tok[i + k])), hnorm(h_{k-1}[i]) ) ) ),  out_k = mtp_norm(h_k)

and shares the embedding table and the output head with the main model; its target is the label
``k`` positions ahead.  Shifts never cross a packed-document boundary (positions restart there):
such slots, and the tail, feed token 0 with a zeroed previous hidden state and carry the ignore
label.  The loss is ``main + mtp_scale * mean_k(depth_k)``, every term a token sum divided by the
global number of valid tokens.  Each depth goes through the chunked fused lm_head + cross entropy
like the main output, so no logits tensor beyond one chunk exists.

Parity: torchtitan/models/deepseek_v3/mtp.py:32-406 (``roll_mtp_sequence``, ``MTPTransformerBlock``,
``MTPDecoder``, ``MTPLoss``).  Not supported with pipeline, context or tensor parallelism (the
reference excludes the first two as well).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from torchtitan_b200.components.loss import IGNORE_INDEX, BaseLoss
from torchtitan_b200.models.common.attention import AttentionContext
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.layers import Linear, RMSNorm
from torchtitan_b200.models.common.module import ModuleDict

__all__ = ["roll_mtp_sequence", "MTPBlock", "MTPDecoder", "MTPLoss"]


def roll_mtp_sequence(sequence: torch.Tensor, *, shift: int, fill_value, positions: torch.Tensor | None = None,
                      return_valid_mask: bool = False):
    """``out[i] = sequence[i + shift]`` along dim 0 where that stays inside the document of ``i``
    (``positions[i + shift] == positions[i] + shift``), ``fill_value`` elsewhere."""
    n = sequence.shape[0]
    if shift <= 0 or shift > n:
        raise ValueError(f"MTP roll shift must be in [1, {n}], got {shift}")
    rolled = torch.full_like(sequence, fill_value)
    valid = torch.zeros(n, dtype=torch.bool, device=sequence.device)
    if positions is None:
        valid[: n - shift] = True
    else:
        if positions.shape[0] < n:
            raise ValueError(f"MTP positions need at least {n} tokens, got {positions.shape[0]}")
        valid[: n - shift] = positions[shift:n] == positions[: n - shift] + shift
    src = sequence[shift:]
    mask = valid[: n - shift].reshape(-1, *([1] * (sequence.dim() - 1)))
    rolled[: n - shift] = torch.where(mask, src, rolled[: n - shift])
    return (rolled, valid) if return_valid_mask else rolled


class MTPBlock(TransformerBlock):
    @dataclass(kw_only=True, slots=True)
    class Config(TransformerBlock.Config):
        dim: int = 0
        enorm: RMSNorm.Config = field(default_factory=RMSNorm.Config)
        hnorm: RMSNorm.Config = field(default_factory=RMSNorm.Config)
        eh_proj: Linear.Config = field(default_factory=Linear.Config)
        mtp_norm: RMSNorm.Config = field(default_factory=RMSNorm.Config)

    def __init__(self, config: "MTPBlock.Config", **_):
        super().__init__(config)
        c = config
        for n in (c.enorm, c.hnorm, c.mtp_norm):
            n.dim = c.dim
        c.eh_proj.in_features, c.eh_proj.out_features = 2 * c.dim, c.dim
        self.enorm, self.hnorm, self.mtp_norm = c.enorm.build(), c.hnorm.build(), c.mtp_norm.build()
        self.eh_proj = c.eh_proj.build()

    def forward(self, input_embed: torch.Tensor, prev_hidden: torch.Tensor, valid: torch.Tensor,  # type: ignore[override]
                positions: torch.Tensor, ctx: AttentionContext | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(hidden state for the next depth, normed output for the head)``."""
        prev_hidden = prev_hidden * valid.unsqueeze(-1).to(prev_hidden.dtype)
        h = self.eh_proj(torch.cat([self.enorm(input_embed), self.hnorm(prev_hidden)], dim=-1))
        h = TransformerBlock.forward(self, h, positions, ctx)
        return h, self.mtp_norm(h)


class MTPDecoder(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        mtp_layers: list = field(default_factory=list)   # list[MTPBlock.Config]
        mtp_scale: float = 0.3

        def update_from_config(self, *, trainer_config=None, **kw) -> None:
            n_main = len(self.layers)
            self.layers.extend(self.mtp_layers)     # the context-length update reaches the MTP blocks too
            try:
                Decoder.Config.update_from_config(self, trainer_config=trainer_config, **kw)
            finally:
                del self.layers[n_main:]
            if trainer_config is not None and self.mtp_layers:
                par = trainer_config.parallelism
                for name in ("pipeline_parallel_degree", "context_parallel_degree", "tensor_parallel_degree"):
                    if getattr(par, name, 1) > 1:
                        raise NotImplementedError(f"multi-token prediction does not support {name} > 1")

    def __init__(self, config: "MTPDecoder.Config", **_):
        super().__init__(config)
        for blk in config.mtp_layers:
            blk.dim = config.dim
        self.mtp_layers = ModuleDict({str(i): blk.build() for i, blk in enumerate(config.mtp_layers)}) \
            if config.mtp_layers else None
        if config.trainable_param_pattern and self.mtp_layers is not None:
            import re

            pat = re.compile(config.trainable_param_pattern)
            for n, p in self.named_parameters():
                if not pat.search(n):
                    p.requires_grad_(False)

    def forward(self, tokens, positions=None, ctx=None, *, return_hidden: bool = False):
        """Without MTP layers: the plain decoder.  With them: a list, the main output followed by
        one output per depth (hidden states when ``return_hidden``, logits otherwise)."""
        if self.mtp_layers is None:
            return super().forward(tokens, positions, ctx, return_hidden=return_hidden)
        if positions is None:
            positions = torch.arange(tokens.shape[0], device=tokens.device)
        if ctx is None:
            ctx = self.build_context(positions)
        h = self.tok_embeddings(tokens)
        for layer in self.layers.values():
            h = layer(h, positions, ctx)
        outs = [self.norm(h)]
        prev = h        # the depths consume the last block's output before the final norm
        for depth, layer in enumerate(self.mtp_layers.values(), 1):
            mtp_tokens, valid = roll_mtp_sequence(tokens, shift=depth, fill_value=0, positions=positions,
                                                  return_valid_mask=True)
            prev, out = layer(self.tok_embeddings(mtp_tokens), prev, valid, positions, ctx)
            outs.append(out)
        if return_hidden:
            return outs
        return [self.lm_head(o) for o in outs]


class MTPLoss(BaseLoss):
    """``main + mtp_scale * mean over depths``; ``inner`` is the per-output loss (token sum divided
    by the global valid-token count), called once per output so that the chunked fused loss applies
    to every depth."""

    needs_positions = True

    def __init__(self, inner: BaseLoss, mtp_scale: float = 0.3):
        super().__init__(getattr(inner, "config", None))
        self.inner = inner
        self.mtp_scale = mtp_scale
        self.needs_hidden = getattr(inner, "needs_hidden", False)

    def __getattr__(self, name):      # set_lm_head and friends go to the wrapped loss
        return getattr(self.__dict__["inner"], name)

    def __call__(self, pred, labels, global_valid_tokens, positions=None):
        if not isinstance(pred, (list, tuple)):
            return self.inner(pred, labels, global_valid_tokens)
        if len(pred) < 2:
            raise ValueError("MTPLoss expects the main prediction followed by one per MTP depth")
        if positions is None:
            raise ValueError("MTPLoss needs the positions to keep shifted labels inside their documents")
        loss = self.inner(pred[0], labels, global_valid_tokens)
        depth_sum = None
        for k, p in enumerate(pred[1:], 1):
            lk = self.inner(p, roll_mtp_sequence(labels, shift=k, fill_value=IGNORE_INDEX, positions=positions),
                            global_valid_tokens)
            depth_sum = lk if depth_sum is None else depth_sum + lk
        return loss + depth_sum * (self.mtp_scale / (len(pred) - 1))
