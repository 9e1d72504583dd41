"""Flux rectified-flow transformer: double-stream blocks (image and text tokens keep separate
weights and meet in one attention), single-stream blocks (fused attention + MLP), AdaLN modulation
from the timestep / pooled-text vector, QK RMSNorm and N-d rotary position embedding.
Parity: torchtitan/models/flux/model/layers.py and model.py:35-250.  Tensors are batched
``[B, L, D]`` (images are not folded into one token stream).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200.models.common.module import Module

__all__ = ["FluxModel", "timestep_embedding", "rope_nd", "apply_rope_nd"]


def timestep_embedding(t: torch.Tensor, dim: int, max_period: int = 10000, time_factor: float = 1000.0) -> torch.Tensor:
    t = time_factor * t.float()
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def rope_nd(ids: torch.Tensor, axes_dim: tuple, theta: float) -> torch.Tensor:
    """``ids [B, L, n_axes]`` -> angles ``[B, L, sum(axes_dim) / 2]``."""
    out = []
    for i, d in enumerate(axes_dim):
        scale = torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d
        omega = 1.0 / (theta ** scale)
        out.append(ids[..., i].double()[..., None] * omega)
    return torch.cat(out, dim=-1).float()


def apply_rope_nd(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent pairs of ``x [B, H, L, D]`` by ``ang [B, L, D/2]``."""
    xr = x.float().reshape(*x.shape[:-1], -1, 2)
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    out = torch.stack([xr[..., 0] * c - xr[..., 1] * s, xr[..., 0] * s + xr[..., 1] * c], dim=-1)
    return out.reshape(x.shape).to(x.dtype)


def _attention(q, k, v, ang):
    q, k = apply_rope_nd(q, ang), apply_rope_nd(k, ang)
    o = F.scaled_dot_product_attention(q, k, v)
    return o.transpose(1, 2).reshape(o.shape[0], o.shape[2], -1)


class _QKNorm(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.q = nn.Parameter(torch.ones(dim))
        self.k = nn.Parameter(torch.ones(dim))

    def forward(self, q, k):
        return F.rms_norm(q, (q.shape[-1],), self.q, 1e-6), F.rms_norm(k, (k.shape[-1],), self.k, 1e-6)


class _Modulation(nn.Module):
    def __init__(self, dim, n):
        super().__init__()
        self.n = n
        self.lin = nn.Linear(dim, n * dim)

    def forward(self, vec):
        return self.lin(F.silu(vec))[:, None, :].chunk(self.n, dim=-1)


class _StreamHalf(nn.Module):
    """One side (image or text) of a double-stream block."""

    def __init__(self, h, heads, mlp_hidden, qkv_bias):
        super().__init__()
        self.mod = _Modulation(h, 6)
        self.norm1 = nn.LayerNorm(h, elementwise_affine=False, eps=1e-6)
        self.qkv = nn.Linear(h, 3 * h, bias=qkv_bias)
        self.qk_norm = _QKNorm(h // heads)
        self.proj = nn.Linear(h, h)
        self.norm2 = nn.LayerNorm(h, elementwise_affine=False, eps=1e-6)
        self.mlp = nn.Sequential(nn.Linear(h, mlp_hidden), nn.GELU(approximate="tanh"), nn.Linear(mlp_hidden, h))
        self.heads = heads

    def qkv_of(self, x, shift, scale):
        B, L, _ = x.shape
        qkv = self.qkv((1 + scale) * self.norm1(x) + shift).view(B, L, 3, self.heads, -1).permute(2, 0, 3, 1, 4)
        q, k = self.qk_norm(qkv[0], qkv[1])
        return q, k, qkv[2]


class DoubleStreamBlock(nn.Module):
    def __init__(self, h, heads, mlp_ratio, qkv_bias):
        super().__init__()
        self.img = _StreamHalf(h, heads, int(h * mlp_ratio), qkv_bias)
        self.txt = _StreamHalf(h, heads, int(h * mlp_ratio), qkv_bias)

    def forward(self, img, txt, vec, ang):
        im, tm = self.img.mod(vec), self.txt.mod(vec)
        iq, ik, iv = self.img.qkv_of(img, im[0], im[1])
        tq, tk, tv = self.txt.qkv_of(txt, tm[0], tm[1])
        o = _attention(torch.cat([tq, iq], 2), torch.cat([tk, ik], 2), torch.cat([tv, iv], 2), ang)
        to, io = o[:, :txt.shape[1]], o[:, txt.shape[1]:]
        img = img + im[2] * self.img.proj(io)
        img = img + im[5] * self.img.mlp((1 + im[4]) * self.img.norm2(img) + im[3])
        txt = txt + tm[2] * self.txt.proj(to)
        txt = txt + tm[5] * self.txt.mlp((1 + tm[4]) * self.txt.norm2(txt) + tm[3])
        return img, txt


class SingleStreamBlock(nn.Module):
    def __init__(self, h, heads, mlp_ratio):
        super().__init__()
        self.heads, self.h, self.mlp_hidden = heads, h, int(h * mlp_ratio)
        self.mod = _Modulation(h, 3)
        self.norm = nn.LayerNorm(h, elementwise_affine=False, eps=1e-6)
        self.linear1 = nn.Linear(h, 3 * h + self.mlp_hidden)
        self.linear2 = nn.Linear(h + self.mlp_hidden, h)
        self.qk_norm = _QKNorm(h // heads)

    def forward(self, x, vec, ang):
        shift, scale, gate = self.mod(vec)
        B, L, _ = x.shape
        qkv, mlp = self.linear1((1 + scale) * self.norm(x) + shift).split([3 * self.h, self.mlp_hidden], dim=-1)
        qkv = qkv.view(B, L, 3, self.heads, -1).permute(2, 0, 3, 1, 4)
        q, k = self.qk_norm(qkv[0], qkv[1])
        o = _attention(q, k, qkv[2], ang)
        return x + gate * self.linear2(torch.cat([o, F.gelu(mlp, approximate="tanh")], dim=-1))


class FluxModel(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        in_channels: int = 64
        out_channels: int = 64
        vec_in_dim: int = 768
        context_in_dim: int = 4096
        hidden_size: int = 3072
        mlp_ratio: float = 4.0
        num_heads: int = 24
        depth: int = 19
        depth_single_blocks: int = 38
        axes_dim: tuple = (16, 56, 56)
        theta: int = 10_000
        qkv_bias: bool = True

        def get_nparams_and_flops(self, model, seq_len: int):
            n = sum(p.numel() for p in model.parameters())
            return n, 6 * n + 6 * (self.depth + self.depth_single_blocks) * self.hidden_size * seq_len

    def __init__(self, config: "FluxModel.Config", **_):
        super().__init__(config)
        c = config
        h = c.hidden_size
        assert sum(c.axes_dim) == h // c.num_heads, "axes_dim must sum to the head dimension"
        self.img_in = nn.Linear(c.in_channels, h)
        self.txt_in = nn.Linear(c.context_in_dim, h)
        self.time_in = nn.Sequential(nn.Linear(256, h), nn.SiLU(), nn.Linear(h, h))
        self.vector_in = nn.Sequential(nn.Linear(c.vec_in_dim, h), nn.SiLU(), nn.Linear(h, h))
        self.double_blocks = nn.ModuleList(DoubleStreamBlock(h, c.num_heads, c.mlp_ratio, c.qkv_bias) for _ in range(c.depth))
        self.single_blocks = nn.ModuleList(SingleStreamBlock(h, c.num_heads, c.mlp_ratio) for _ in range(c.depth_single_blocks))
        self.final_norm = nn.LayerNorm(h, elementwise_affine=False, eps=1e-6)
        self.final_mod = nn.Linear(h, 2 * h)
        self.final_linear = nn.Linear(h, c.out_channels)

    def init_states(self, seed: int = 0, **_) -> None:
        g = torch.Generator().manual_seed(seed)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                with torch.no_grad():
                    m.weight.copy_(torch.empty(m.weight.shape).normal_(0, 0.02, generator=g))
                    if m.bias is not None:
                        m.bias.zero_()
        for m in (self.final_mod, self.final_linear):   # the model starts as the zero map
            nn.init.zeros_(m.weight)

    def forward(self, img, img_ids, txt, txt_ids, timesteps, y):
        """``img [B, L_img, C]`` latent patches, ``txt [B, L_txt, context]`` T5 states, ``y [B, vec]`` pooled CLIP
        vector, ``timesteps [B]`` in [0, 1]; returns the predicted velocity ``[B, L_img, C]``."""
        c = self.config
        img, txt = self.img_in(img), self.txt_in(txt)
        vec = self.time_in(timestep_embedding(timesteps, 256).to(img.dtype)) + self.vector_in(y)
        ang = rope_nd(torch.cat([txt_ids, img_ids], dim=1), c.axes_dim, c.theta)
        for blk in self.double_blocks:
            img, txt = blk(img, txt, vec, ang)
        x = torch.cat([txt, img], dim=1)
        for blk in self.single_blocks:
            x = blk(x, vec, ang)
        x = x[:, txt.shape[1]:]
        shift, scale = self.final_mod(F.silu(vec))[:, None, :].chunk(2, dim=-1)
        return self.final_linear((1 + scale) * self.final_norm(x) + shift)
