"""Image generation with a trained Flux model: shifted time schedule, Euler integration of the
learned velocity field from noise (t = 1) to data (t = 0), optional classifier-free guidance,
latent unpacking, autoencoder decoding and image export.

Parity: torchtitan/models/flux/inference/sampling.py:34-257 (``time_shift``, ``get_schedule``,
``generate_image``, ``denoise``, ``save_image``) and flux/utils.py (latent packing, position ids).
"""

from __future__ import annotations

import math
import os

import torch

from .trainer import make_ids, pack_latents

__all__ = ["time_shift", "get_schedule", "unpack_latents", "denoise", "generate_image", "save_image"]


def time_shift(mu: float, sigma: float, t: torch.Tensor) -> torch.Tensor:
    return math.exp(mu) / (math.exp(mu) + (1 / t - 1) ** sigma)


def get_schedule(num_steps: int, image_seq_len: int, base_shift: float = 0.5, max_shift: float = 1.15,
                 shift: bool = True) -> list[float]:
    """``num_steps + 1`` times from 1 to 0; with ``shift`` the schedule spends more steps at high
    noise for longer latent sequences (``mu`` is linear in the sequence length through the points
    (256, base_shift) and (4096, max_shift))."""
    t = torch.linspace(1, 0, num_steps + 1)
    if shift:
        m = (max_shift - base_shift) / (4096 - 256)
        mu = m * image_seq_len + (base_shift - m * 256)
        t = time_shift(mu, 1.0, t)
    return t.tolist()


def unpack_latents(x: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """Inverse of ``pack_latents``: ``[B, (h/2)(w/2), 4 C]`` -> ``[B, C, h, w]``."""
    B, _, c4 = x.shape
    C = c4 // 4
    return x.view(B, h // 2, w // 2, C, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, C, h, w)


@torch.no_grad()
def denoise(model, *, latent_channels: int, img_height: int, img_width: int, steps: int, txt: torch.Tensor, vec: torch.Tensor,
            empty_txt: torch.Tensor | None = None, empty_vec: torch.Tensor | None = None, guidance_scale: float | None = None,
            generator: torch.Generator | None = None, downsample: int = 8) -> torch.Tensor:
    """Latents ``[B, C, H/8, W/8]`` sampled for the given text conditioning."""
    dev, dt = txt.device, txt.dtype
    B = txt.shape[0]
    lh, lw = 2 * math.ceil(img_height / (2 * downsample)), 2 * math.ceil(img_width / (2 * downsample))
    z = torch.randn(B, latent_channels, lh, lw, generator=generator, device=dev, dtype=dt)
    cfg = guidance_scale is not None and empty_txt is not None
    if cfg:
        if empty_vec is None:
            raise ValueError("classifier-free guidance needs the empty-prompt encodings of both encoders")
        z = torch.cat([z, z])
        txt, vec = torch.cat([empty_txt, txt]), torch.cat([empty_vec, vec])
    n = z.shape[0]
    img_ids, txt_ids = make_ids(n, lh // 2, lw // 2, txt.shape[1], dev)
    x = pack_latents(z)
    times = get_schedule(steps, (lh // 2) * (lw // 2))
    for t_cur, t_next in zip(times[:-1], times[1:]):
        v = model(x, img_ids, txt, txt_ids, torch.full((n,), t_cur, device=dev, dtype=dt), vec)
        if cfg:
            vu, vc = v.chunk(2)
            v = (vu + guidance_scale * (vc - vu)).repeat(2, 1, 1)
        x = x + (t_next - t_cur) * v
    if cfg:
        x = x.chunk(2)[1]
    return unpack_latents(x, lh, lw)


@torch.no_grad()
def generate_image(model, autoencoder, *, txt: torch.Tensor, vec: torch.Tensor, img_height: int, img_width: int, steps: int = 50,
                   empty_txt=None, empty_vec=None, guidance_scale: float | None = None, generator=None) -> torch.Tensor:
    """``[B, 3, H, W]`` images in [-1, 1]."""
    z = denoise(model, latent_channels=autoencoder.config.z_channels, img_height=img_height, img_width=img_width, steps=steps,
                txt=txt, vec=vec, empty_txt=empty_txt, empty_vec=empty_vec, guidance_scale=guidance_scale,
                generator=generator, downsample=autoencoder.downsample_factor)
    return autoencoder.decode(z.to(next(autoencoder.parameters()).dtype))


def save_image(x: torch.Tensor, path: str) -> str:
    """First image of the batch as an 8-bit file: PNG / JPEG through PIL when it is installed,
    binary PPM (same pixels, no dependency) otherwise."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    img = ((x[0].clamp(-1, 1) + 1.0) * 127.5).permute(1, 2, 0).round().to(torch.uint8).cpu().contiguous()
    try:
        from PIL import Image

        Image.fromarray(img.numpy()).save(path)
        return path
    except ImportError:
        path = os.path.splitext(path)[0] + ".ppm"
        with open(path, "wb") as f:
            f.write(f"P6 {img.shape[1]} {img.shape[0]} 255\n".encode())
            f.write(img.numpy().tobytes())
        return path
