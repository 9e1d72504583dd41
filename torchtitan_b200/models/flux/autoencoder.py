"""Flux's latent autoencoder: a convolutional VAE that maps ``[B, 3, H, W]`` images in [-1, 1] to
``[B, z, H/8, W/8]`` latents and back.

Encoder: 3x3 stem, one stage per entry of ``ch_mult`` (``num_res_blocks`` residual blocks, then a
stride-2 convolution with asymmetric right/bottom padding on all but the last stage), a middle of
residual block / single-head spatial self-attention / residual block, group norm, SiLU and a 3x3
head producing mean and log-variance.  Decoder: the mirror image with ``num_res_blocks + 1`` blocks
per stage and nearest-neighbour 2x upsampling followed by a 3x3 convolution.  Latents are
``(z - shift_factor) * scale_factor`` on the way out of ``encode`` and the inverse into ``decode``.

Parity: torchtitan/models/flux/model/autoencoder.py:27-435 (same module tree and parameter names:
``encoder.down.<i>.block.<j>``, ``mid.block_1 / attn_1 / block_2``, ``decoder.up.<i>...``; weights of
the released ``ae.safetensors`` load by name).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from torchtitan_b200.models.common.module import Module

__all__ = ["AutoEncoder"]


def _gn(ch: int) -> nn.GroupNorm:
    return nn.GroupNorm(num_groups=32 if ch % 32 == 0 else ch, num_channels=ch, eps=1e-6, affine=True)


class _Res(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.norm1, self.conv1 = _gn(cin), nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = _gn(cout), nn.Conv2d(cout, cout, 3, padding=1)
        self.nin_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return (x if self.nin_shortcut is None else self.nin_shortcut(x)) + h


class _Attn(nn.Module):
    """Single-head self-attention over the ``H * W`` positions (1x1 convolutions as projections)."""

    def __init__(self, ch: int):
        super().__init__()
        self.norm = _gn(ch)
        self.q, self.k, self.v, self.proj_out = (nn.Conv2d(ch, ch, 1) for _ in range(4))

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.norm(x)
        q, k, v = (f(h).reshape(B, 1, C, H * W).transpose(2, 3) for f in (self.q, self.k, self.v))
        o = F.scaled_dot_product_attention(q, k, v).transpose(2, 3).reshape(B, C, H, W)
        return x + self.proj_out(o)


class _Down(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.conv = nn.Conv2d(ch, ch, 3, stride=2, padding=0)

    def forward(self, x):
        return self.conv(F.pad(x, (0, 1, 0, 1)))


class _Up(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.conv = nn.Conv2d(ch, ch, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class _Stage(nn.Module):
    def __init__(self, blocks: list[nn.Module], resample: nn.Module | None, down: bool):
        super().__init__()
        self.block = nn.ModuleList(blocks)
        self.attn = nn.ModuleList()
        if resample is not None:
            setattr(self, "downsample" if down else "upsample", resample)


class _Mid(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.block_1, self.attn_1, self.block_2 = _Res(ch, ch), _Attn(ch), _Res(ch, ch)

    def forward(self, x):
        return self.block_2(self.attn_1(self.block_1(x)))


class _Encoder(nn.Module):
    def __init__(self, c: "AutoEncoder.Config"):
        super().__init__()
        self.conv_in = nn.Conv2d(c.in_channels, c.ch, 3, padding=1)
        mult = (1,) + tuple(c.ch_mult)
        stages = []
        cur = c.ch
        for i in range(len(c.ch_mult)):
            cin, cout = c.ch * mult[i], c.ch * c.ch_mult[i]
            blocks = [_Res(cin if j == 0 else cout, cout) for j in range(c.num_res_blocks)]
            cur = cout
            stages.append(_Stage(blocks, _Down(cur) if i != len(c.ch_mult) - 1 else None, down=True))
        self.down = nn.ModuleList(stages)
        self.mid = _Mid(cur)
        self.norm_out, self.conv_out = _gn(cur), nn.Conv2d(cur, 2 * c.z_channels, 3, padding=1)

    def forward(self, x):
        h = self.conv_in(x)
        for st in self.down:
            for b in st.block:
                h = b(h)
            if hasattr(st, "downsample"):
                h = st.downsample(h)
        return self.conv_out(F.silu(self.norm_out(self.mid(h))))


class _Decoder(nn.Module):
    def __init__(self, c: "AutoEncoder.Config"):
        super().__init__()
        n = len(c.ch_mult)
        cur = c.ch * c.ch_mult[-1]
        self.conv_in = nn.Conv2d(c.z_channels, cur, 3, padding=1)
        self.mid = _Mid(cur)
        stages: list[nn.Module] = [None] * n   # type: ignore[list-item]
        for i in reversed(range(n)):
            cout = c.ch * c.ch_mult[i]
            blocks = [_Res(cur if j == 0 else cout, cout) for j in range(c.num_res_blocks + 1)]
            cur = cout
            stages[i] = _Stage(blocks, _Up(cur) if i != 0 else None, down=False)
        self.up = nn.ModuleList(stages)      # indexed by resolution level, applied from the last to the first
        self.norm_out, self.conv_out = _gn(cur), nn.Conv2d(cur, c.out_ch, 3, padding=1)

    def forward(self, z):
        h = self.mid(self.conv_in(z))
        for st in reversed(self.up):
            for b in st.block:
                h = b(h)
            if hasattr(st, "upsample"):
                h = st.upsample(h)
        return self.conv_out(F.silu(self.norm_out(h)))


class AutoEncoder(Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        resolution: int = 256
        in_channels: int = 3
        ch: int = 128
        out_ch: int = 3
        ch_mult: tuple[int, ...] = (1, 2, 4, 4)
        num_res_blocks: int = 2
        z_channels: int = 16
        scale_factor: float = 0.3611
        shift_factor: float = 0.1159
        sample: bool = True

    def __init__(self, config: "AutoEncoder.Config", **_):
        super().__init__(config)
        self.encoder, self.decoder = _Encoder(config), _Decoder(config)

    @property
    def downsample_factor(self) -> int:
        return 2 ** (len(self.config.ch_mult) - 1)

    def init_states(self, seed: int = 0, prefix: str = "") -> None:
        """PyTorch's default convolution / norm initialisation under a fixed seed (the released
        weights replace it for real use)."""
        g = torch.random.get_rng_state()
        torch.manual_seed(seed)
        for m in self.modules():
            if hasattr(m, "reset_parameters"):
                m.reset_parameters()
        torch.random.set_rng_state(g)

    def encode(self, x: torch.Tensor, generator: torch.Generator | None = None) -> torch.Tensor:
        mean, logvar = self.encoder(x).chunk(2, dim=1)
        z = mean
        if self.config.sample:
            z = mean + torch.exp(0.5 * logvar) * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)
        return self.config.scale_factor * (z - self.config.shift_factor)

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(z / self.config.scale_factor + self.config.shift_factor)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.decode(self.encode(x))

    def load_released_weights(self, path: str) -> None:
        """Load ``ae.safetensors`` (names match this module tree)."""
        from safetensors.torch import load_file

        missing, unexpected = self.load_state_dict(load_file(path), strict=False)
        if missing or unexpected:
            raise ValueError(f"autoencoder checkpoint mismatch: missing {missing[:4]}, unexpected {unexpected[:4]}")
