"""Vision tower shared by the multimodal flavors: a pre-norm ViT over packed image patches.

Input: ``patches[N, C * P * P]`` (all images of the batch concatenated, row-major over each
image's ``gh x gw`` patch grid) and ``grid_hw[num_images, 2]``.  Patches are embedded by one linear
layer, rotated with a 2-D rotary embedding (half of each head follows the patch row, half the
column), attend bidirectionally *within their own image* (block-diagonal: each image is one
non-causal attention call), and are finally merged ``m x m`` spatially and
projected to the language model's width by a two-layer MLP.  Output: ``[sum_i gh_i gw_i / m^2,
text_dim]`` in image order, plus the per-image token counts.

Parity: torchtitan/models/common/vision_encoder.py:42-180 (block-diagonal mask, ``VisionMLP``,
``VisionAttention``, ``VisionTransformerBlock``) and the per-model towers built from them
(qwen3_5/model.py, kimi_k2_7, muse_glimmer).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200.ops import functional as OF

from .layers import Linear
from .module import InitSpec, Module, ModuleDict, set_init

__all__ = ["VisionEncoder", "VisionBlock", "rope_2d"]


def _layer_norm(dim: int, eps: float) -> nn.LayerNorm:
    ln = nn.LayerNorm(dim, eps=eps)
    set_init(ln.weight, InitSpec(kind="ones"))
    set_init(ln.bias, InitSpec(kind="zeros"))
    return ln


def rope_2d(x: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor, theta: float = 10000.0) -> torch.Tensor:
    """Rotate-half RoPE on ``x[N, H, D]``: the first ``D / 2`` channels by the patch row, the rest
    by the patch column."""
    N, H, D = x.shape
    q = D // 4
    inv = 1.0 / (theta ** (torch.arange(q, device=x.device, dtype=torch.float32) / q))
    ang = torch.cat([rows.float()[:, None] * inv, cols.float()[:, None] * inv], dim=1)      # [N, D/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    a, b = xf[..., : D // 2], xf[..., D // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class VisionBlock(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        dim: int = 0
        num_heads: int = 0
        mlp_dim: int = 0
        norm_eps: float = 1e-6
        wqkv: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))
        proj: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))
        fc1: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))
        fc2: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))

    def __init__(self, config: "VisionBlock.Config", **_):
        super().__init__(config)
        c = config
        if c.dim % c.num_heads or (c.dim // c.num_heads) % 4:
            raise ValueError("vision dim must divide into heads whose size is a multiple of 4")
        self.num_heads, self.head_dim = c.num_heads, c.dim // c.num_heads
        c.wqkv.in_features, c.wqkv.out_features = c.dim, 3 * c.dim
        c.proj.in_features, c.proj.out_features = c.dim, c.dim
        c.fc1.in_features, c.fc1.out_features = c.dim, c.mlp_dim
        c.fc2.in_features, c.fc2.out_features = c.mlp_dim, c.dim
        self.norm1 = _layer_norm(c.dim, c.norm_eps)
        self.norm2 = _layer_norm(c.dim, c.norm_eps)
        self.wqkv, self.proj = c.wqkv.build(), c.proj.build()
        self.fc1, self.fc2 = c.fc1.build(), c.fc2.build()

    def forward(self, x: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor, spans: list[tuple[int, int]]) -> torch.Tensor:
        N = x.shape[0]
        qkv = self.wqkv(self.norm1(x)).view(N, 3, self.num_heads, self.head_dim)
        q, k, v = rope_2d(qkv[:, 0], rows, cols), rope_2d(qkv[:, 1], rows, cols), qkv[:, 2]
        scale = self.head_dim ** -0.5
        outs = [OF.attention(q[a:b].contiguous(), k[a:b].contiguous(), v[a:b].contiguous(), scale=scale, causal=False)
                for a, b in spans]      # block diagonal: an image attends to itself only
        x = x + self.proj(torch.cat(outs, dim=0).reshape(N, -1))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x)), approximate="tanh"))


class VisionEncoder(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        patch_size: int = 14
        in_channels: int = 3
        dim: int = 0
        num_heads: int = 0
        mlp_dim: int = 0
        n_layers: int = 0
        spatial_merge: int = 2
        temporal_patch_size: int = 1
        """Frames per patch: a patch vector holds ``C * temporal_patch_size * P * P`` values (still images repeat the frame)."""
        num_position_embeddings: int = 0
        """Learned position table of ``sqrt(n) x sqrt(n)`` entries, bilinearly interpolated to every image's patch grid
        and added to the patch embeddings (0: rotary positions only)."""
        out_dim: int = 0          # the language model's width
        norm_eps: float = 1e-6
        layers: list = field(default_factory=list)   # list[VisionBlock.Config], filled from the sizes when empty
        patch_embed: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))
        merger_fc1: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))
        merger_fc2: Linear.Config = field(default_factory=lambda: Linear.Config(bias=True))

    def __init__(self, config: "VisionEncoder.Config", **_):
        super().__init__(config)
        c = config
        if not c.layers:
            c.layers = [VisionBlock.Config(dim=c.dim, num_heads=c.num_heads, mlp_dim=c.mlp_dim, norm_eps=c.norm_eps)
                        for _ in range(c.n_layers)]
        m2 = c.spatial_merge ** 2
        c.patch_embed.in_features = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        c.patch_embed.out_features = c.dim
        self.pos_embed = None
        if c.num_position_embeddings:
            side = int(round(c.num_position_embeddings ** 0.5))
            if side * side != c.num_position_embeddings:
                raise ValueError("num_position_embeddings must be a square")
            self.pos_embed = nn.Parameter(torch.empty(c.num_position_embeddings, c.dim))
            set_init(self.pos_embed, InitSpec(kind="normal", std=0.02))
        c.merger_fc1.in_features, c.merger_fc1.out_features = c.dim * m2, c.dim * m2
        c.merger_fc2.in_features, c.merger_fc2.out_features = c.dim * m2, c.out_dim
        self.patch_embed = c.patch_embed.build()
        self.layers = ModuleDict({str(i): b.build() for i, b in enumerate(c.layers)})
        self.norm = _layer_norm(c.dim, c.norm_eps)
        self.merger_fc1, self.merger_fc2 = c.merger_fc1.build(), c.merger_fc2.build()

    def _interpolated_positions(self, h: int, w: int) -> torch.Tensor:
        """The learned ``side x side`` table sampled bilinearly on an ``h x w`` grid that spans it corner to corner
        (row-major ``[h * w, dim]``)."""
        table = self.pos_embed
        side = int(round(table.shape[0] ** 0.5))
        dev = table.device
        ys = torch.linspace(0, side - 1, h, device=dev)
        xs = torch.linspace(0, side - 1, w, device=dev)
        y0, x0 = ys.long(), xs.long()
        y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
        dy, dx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
        t = table.float().view(side, side, -1)
        out = (t[y0][:, x0] * (1 - dy) * (1 - dx) + t[y0][:, x1] * (1 - dy) * dx
               + t[y1][:, x0] * dy * (1 - dx) + t[y1][:, x1] * dy * dx)
        return out.reshape(h * w, -1)

    def tokens_per_image(self, grid_hw: torch.Tensor) -> torch.Tensor:
        m = self.config.spatial_merge
        return (grid_hw[:, 0] // m) * (grid_hw[:, 1] // m)

    def forward(self, patches: torch.Tensor, grid_hw: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``patches[N, C P P]``, ``grid_hw[I, 2]`` (host or device ints) -> ``(embeds[M, out_dim], tokens_per_image[I])``."""
        c = self.config
        m = c.spatial_merge
        grid = [(int(h), int(w)) for h, w in grid_hw.tolist()]
        if any(h % m or w % m for h, w in grid):
            raise ValueError(f"every image grid must be a multiple of the spatial merge size {m}: {grid}")
        dev = patches.device
        rows = torch.cat([torch.arange(h, device=dev).repeat_interleave(w) for h, w in grid])
        cols = torch.cat([torch.arange(w, device=dev).repeat(h) for h, w in grid])
        spans, o = [], 0
        for h, w in grid:
            spans.append((o, o + h * w))
            o += h * w
        if o != patches.shape[0]:
            raise ValueError(f"grid_hw describes {o} patches, got {patches.shape[0]}")
        per_frame = c.in_channels * c.patch_size ** 2
        if c.temporal_patch_size > 1 and patches.shape[1] == per_frame:
            # still images: the frame is repeated over the temporal extent of the patch ([C, frames, P, P] layout)
            patches = patches.view(-1, c.in_channels, 1, c.patch_size ** 2).expand(-1, -1, c.temporal_patch_size, -1)
            patches = patches.reshape(-1, per_frame * c.temporal_patch_size)
        x = self.patch_embed(patches.to(self.patch_embed.weight.dtype))
        if self.pos_embed is not None:
            x = x + torch.cat([self._interpolated_positions(h, w) for h, w in grid]).to(x.dtype)
        for blk in self.layers.values():
            x = blk(x, rows, cols, spans)
        x = self.norm(x)
        merged = []
        for (a, b), (h, w) in zip(spans, grid):     # m x m neighbourhoods -> one token
            t = x[a:b].view(h // m, m, w // m, m, c.dim).permute(0, 2, 1, 3, 4).reshape((h // m) * (w // m), m * m * c.dim)
            merged.append(t)
        y = self.merger_fc2(F.gelu(self.merger_fc1(torch.cat(merged, dim=0))))
        return y, torch.tensor([(h // m) * (w // m) for h, w in grid], device=dev)
