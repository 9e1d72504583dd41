"""Text decoder with a vision tower: image features replace placeholder tokens.

A sample's token stream carries, for each image, one contiguous run of ``image_token_id`` as long
as the image's feature count (``gh * gw / merge^2``).  ``MultimodalDecoder.forward`` embeds the
tokens, runs the tower on the packed patches, writes the features over the placeholder runs (in
order) and continues as the text decoder.  With ``mrope_sections`` set on the attention layers'
RoPE, rotary positions have three axes (temporal, height, width): text tokens advance all three
together, the tokens of an image share one temporal position and spread over height / width, and
the text after an image continues from the largest position used
(``mrope_position_ids``).  Document masking still follows the 1-D ``positions``.

Parity: torchtitan/models/common/multimodal.py:38-124 (``get_vision_positions``,
``scatter_vision_embeds``), the multimodal decoders of qwen3_5 / kimi_k2_7 / muse_glimmer, and
Qwen-VL's MRoPE index rule.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .attention import AttentionContext
from .decoder import Decoder
from .vision_encoder import VisionEncoder

__all__ = ["get_vision_positions", "scatter_vision_embeds", "mrope_position_ids", "MultimodalDecoder", "to_multimodal"]


def get_vision_positions(tokens: torch.Tensor, tokens_per_item: torch.Tensor, placeholder_id: int) -> list[tuple[int, int, int]]:
    """``(item, start, length)`` of every placeholder run; raises when the runs and the visual
    items disagree in number or length (scattering anyway would corrupt the embeddings)."""
    m = tokens == placeholder_id
    prev = torch.zeros_like(m)
    prev[1:] = m[:-1]
    nxt = torch.zeros_like(m)
    nxt[:-1] = m[1:]
    starts = torch.where(m & ~prev)[0].tolist()
    ends = torch.where(m & ~nxt)[0].tolist()
    want = [int(v) for v in tokens_per_item.tolist()]
    if len(starts) != len(want):
        raise ValueError(f"multimodal misalignment: {len(starts)} run(s) of placeholder id {placeholder_id} in the "
                         f"token sequence, {len(want)} visual item(s)")
    out = []
    for i, (a, b) in enumerate(zip(starts, ends)):
        if b - a + 1 != want[i]:
            raise ValueError(f"multimodal misalignment: placeholder run {i} spans {b - a + 1} token(s), visual item "
                             f"{i} produced {want[i]} embedding(s)")
        out.append((i, a, want[i]))
    return out


def scatter_vision_embeds(inputs_embeds: torch.Tensor, vision_embeds: torch.Tensor,
                          vision_positions: list[tuple[int, int, int]]) -> torch.Tensor:
    """Text embeddings with the packed vision features written over the placeholder runs
    (out of place, differentiable in both arguments)."""
    if not vision_positions:
        return inputs_embeds
    idx = torch.cat([torch.arange(a, a + n, device=inputs_embeds.device) for _, a, n in vision_positions])
    if idx.numel() != vision_embeds.shape[0]:
        raise ValueError(f"placeholder runs consume {idx.numel()} embeddings, the vision tower produced {vision_embeds.shape[0]}")
    return inputs_embeds.index_copy(0, idx, vision_embeds.to(inputs_embeds.dtype))


def mrope_position_ids(tokens: torch.Tensor, positions: torch.Tensor, grid_hw: torch.Tensor, merge: int,
                       placeholder_id: int) -> torch.Tensor:
    """``[3, T]`` rotary positions (temporal, height, width).  Inside each document text tokens
    count up on all axes; an image's tokens keep the temporal index of its first token and add
    their merged-grid row / column to the height / width axes; the next text token continues at
    ``1 + max`` of everything before it."""
    T = tokens.shape[0]
    out = torch.zeros(3, T, dtype=torch.int64)
    tok, pos = tokens.tolist(), positions.tolist()
    grids = [(int(h) // merge, int(w) // merge) for h, w in grid_hw.tolist()]
    gi, i, nxt = 0, 0, 0
    while i < T:
        if pos[i] == 0:
            nxt = 0                     # a new document restarts every axis
        if tok[i] == placeholder_id and gi < len(grids):
            h, w = grids[gi]
            gi += 1
            n = h * w
            r = torch.arange(h).repeat_interleave(w)
            c = torch.arange(w).repeat(h)
            out[0, i:i + n] = nxt
            out[1, i:i + n] = nxt + r[: T - i]
            out[2, i:i + n] = nxt + c[: T - i]
            nxt += max(h, w)
            i += n
        else:
            out[:, i] = nxt
            nxt += 1
            i += 1
    return out.to(tokens.device)


class MultimodalDecoder(Decoder):
    @dataclass(kw_only=True, slots=True)
    class Config(Decoder.Config):
        vision_encoder: VisionEncoder.Config = field(default_factory=VisionEncoder.Config)
        image_token_id: int = 0
        use_mrope: bool = False

    def __init__(self, config: "MultimodalDecoder.Config", **_):
        super().__init__(config)
        config.vision_encoder.out_dim = config.dim
        self.vision_encoder = config.vision_encoder.build()
        if config.trainable_param_pattern:
            import re

            pat = re.compile(config.trainable_param_pattern)
            for n, p in self.vision_encoder.named_parameters():
                if not pat.search("vision_encoder." + n):
                    p.requires_grad_(False)

    def forward(self, tokens, positions=None, ctx: AttentionContext | None = None, *, return_hidden: bool = False,
                pixel_patches: torch.Tensor | None = None, grid_hw: torch.Tensor | None = None):
        if positions is None:
            positions = torch.arange(tokens.shape[0], device=tokens.device)
        if ctx is None:
            ctx = self.build_context(positions)
        h = self.tok_embeddings(tokens)
        if pixel_patches is not None and pixel_patches.shape[0] > 0:
            feats, per_item = self.vision_encoder(pixel_patches, grid_hw)
            h = scatter_vision_embeds(h, feats, get_vision_positions(tokens, per_item, self.config.image_token_id))
            if self.config.use_mrope:
                ctx.rope_positions = mrope_position_ids(tokens, positions, grid_hw, self.config.vision_encoder.spatial_merge,
                                                        self.config.image_token_id)
        elif self.config.use_mrope:
            ctx.rope_positions = positions.unsqueeze(0).expand(3, -1).contiguous()
        for layer in self.layers.values():
            h = layer(h, positions, ctx)
        if self.norm is not None:
            h = self.norm(h)
        if return_hidden or self.lm_head is None:
            return h
        logits = self.lm_head(h)
        if self.config.final_logit_multiplier != 1.0:
            logits = logits * self.config.final_logit_multiplier
        cap = self.config.final_logit_softcap
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits


def to_multimodal(text_cfg: Decoder.Config, vision: VisionEncoder.Config, image_token_id: int,
                  mrope_sections: tuple[int, ...] | None = None, mrope_interleaved: bool = False) -> "MultimodalDecoder.Config":
    """A text decoder config with a vision tower in front; with ``mrope_sections`` every rotary
    attention layer switches to three-axis positions."""
    import dataclasses

    kw = {f.name: getattr(text_cfg, f.name) for f in dataclasses.fields(text_cfg) if not f.name.startswith("_")}
    if mrope_sections is not None:
        for blk in kw["layers"]:
            rope = getattr(blk.attention, "rope", None)
            if rope is not None:
                rope.mrope_sections = tuple(mrope_sections)
                rope.mrope_interleaved = mrope_interleaved
    return MultimodalDecoder.Config(**kw, vision_encoder=vision, image_token_id=image_token_id,
                                    use_mrope=mrope_sections is not None)
