"""Rectified-flow training of the Flux transformer (parity: torchtitan/models/flux/trainer.py).

One step: latents ``x0`` (from the autoencoder; synthetic here), noise ``e``, ``t ~ U(0, 1)``,
``x_t = (1 - t) x0 + t e``; the model predicts the velocity ``e - x0`` and is trained with MSE.
Text conditioning arrives as T5 token states and a pooled CLIP vector; with
``encoders="random"`` both come from small randomly initialised embedding tables (the released
encoders need downloaded weights).  Data parallelism averages gradients over the world group;
AdamW with the framework's warmup / decay schedule.
"""

from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from .model import FluxModel

__all__ = ["FluxTrainer", "flow_matching_batch", "pack_latents", "make_ids"]


def pack_latents(z: torch.Tensor) -> torch.Tensor:
    """``[B, C, H, W]`` autoencoder latents -> ``[B, (H/2)(W/2), 4C]`` patch tokens."""
    B, C, H, W = z.shape
    z = z.view(B, C, H // 2, 2, W // 2, 2).permute(0, 2, 4, 1, 3, 5)
    return z.reshape(B, (H // 2) * (W // 2), C * 4)


def make_ids(B: int, h: int, w: int, l_txt: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    img_ids = torch.zeros(h, w, 3, device=device)
    img_ids[..., 1] = torch.arange(h, device=device)[:, None]
    img_ids[..., 2] = torch.arange(w, device=device)[None, :]
    return img_ids.view(1, h * w, 3).expand(B, -1, -1), torch.zeros(B, l_txt, 3, device=device)


def flow_matching_batch(x0: torch.Tensor, gen: torch.Generator | None = None):
    noise = torch.randn(x0.shape, generator=gen, device=x0.device, dtype=x0.dtype)
    t = torch.rand(x0.shape[0], generator=gen, device=x0.device, dtype=x0.dtype)
    xt = (1 - t[:, None, None]) * x0 + t[:, None, None] * noise
    return xt, t, noise - x0


class FluxTrainer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        model: FluxModel.Config = field(default_factory=FluxModel.Config)
        steps: int = 10
        batch_size: int = 2
        img_size: int = 64          # pixels; the autoencoder downsamples by 8, patches are 2x2 latents
        latent_channels: int = 16
        txt_len: int = 16
        lr: float = 1e-4
        warmup_steps: int = 2
        weight_decay: float = 0.01
        seed: int = 0
        encoders: str = "random"
        dtype: str = "float32"
        log_freq: int = 1
        autoencoder: object | None = None
        """``AutoEncoder.Config``: train on pixels (synthetic images are encoded to latents by the
        frozen autoencoder) instead of on synthetic latents."""
        autoencoder_path: str | None = None
        eval_timesteps: int = 8
        """Validation: the flow-matching loss at this many evenly spaced noise levels."""

    def __init__(self, config: "FluxTrainer.Config", **_):
        super().__init__(config)
        c = config
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.dtype = getattr(torch, c.dtype)
        self.model = c.model.build()
        self.model.init_states(seed=c.seed)
        self.model.to(self.device, self.dtype)
        g = torch.Generator().manual_seed(c.seed + 1)
        self.t5_table = torch.randn(1024, c.model.context_in_dim, generator=g).to(self.device, self.dtype)
        self.clip_table = torch.randn(1024, c.model.vec_in_dim, generator=g).to(self.device, self.dtype)
        self.autoencoder = None
        if c.autoencoder is not None:
            self.autoencoder = c.autoencoder.build()
            self.autoencoder.init_states(seed=c.seed + 2)
            if c.autoencoder_path:
                self.autoencoder.load_released_weights(c.autoencoder_path)
            self.autoencoder.to(self.device, self.dtype).requires_grad_(False).eval()
        self.opt = torch.optim.AdamW(self.model.parameters(), lr=c.lr, weight_decay=c.weight_decay)
        self.sched = torch.optim.lr_scheduler.LambdaLR(
            self.opt, lambda s: min(1.0, (s + 1) / max(1, c.warmup_steps)) * 0.5 * (1 + math.cos(math.pi * min(1.0, s / max(1, c.steps)))))
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed + 17 * (dist.get_rank() if dist.is_initialized() else 0))
        self.losses: list[float] = []

    def synthetic_batch(self):
        c = self.config
        if self.autoencoder is not None:
            img = torch.rand(c.batch_size, 3, c.img_size, c.img_size, generator=self.gen, device=self.device, dtype=self.dtype) * 2 - 1
            with torch.no_grad():
                z = self.autoencoder.encode(img, generator=self.gen)
            lat = z.shape[-1]
        else:
            lat = c.img_size // 8
            z = torch.randn(c.batch_size, c.latent_channels, lat, lat, generator=self.gen, device=self.device, dtype=self.dtype)
        tokens = torch.randint(0, 1024, (c.batch_size, c.txt_len), generator=self.gen, device=self.device)
        return pack_latents(z), self.t5_table[tokens], self.clip_table[tokens[:, 0]], lat // 2

    def train_step(self) -> float:
        x0, txt, y, side = self.synthetic_batch()
        xt, t, target = flow_matching_batch(x0, self.gen)
        img_ids, txt_ids = make_ids(x0.shape[0], side, side, txt.shape[1], self.device)
        pred = self.model(xt, img_ids, txt, txt_ids, t, y)
        loss = nn.functional.mse_loss(pred.float(), target.float())
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        if dist.is_initialized() and dist.get_world_size() > 1:
            for p in self.model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
        torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.opt.step()
        self.sched.step()
        return float(loss.detach())

    @torch.no_grad()
    def validate(self, batches: int = 1) -> float:
        """Mean flow-matching loss over ``eval_timesteps`` fixed noise levels (the stratified
        evaluation of torchtitan/models/flux/validate.py: every sample is scored at each level
        instead of at one random time)."""
        was_training = self.model.training
        self.model.eval()
        tot, n = 0.0, 0
        levels = [(i + 0.5) / self.config.eval_timesteps for i in range(self.config.eval_timesteps)]
        for _ in range(batches):
            x0, txt, y, side = self.synthetic_batch()
            img_ids, txt_ids = make_ids(x0.shape[0], side, side, txt.shape[1], self.device)
            noise = torch.randn(x0.shape, generator=self.gen, device=x0.device, dtype=x0.dtype)
            for tv in levels:
                t = torch.full((x0.shape[0],), tv, device=x0.device, dtype=x0.dtype)
                xt = (1 - tv) * x0 + tv * noise
                pred = self.model(xt, img_ids, txt, txt_ids, t, y)
                tot += float(nn.functional.mse_loss(pred.float(), (noise - x0).float()))
                n += 1
        self.model.train(was_training)
        return tot / max(n, 1)

    @torch.no_grad()
    def generate(self, prompt_tokens: torch.Tensor, *, steps: int = 4, guidance_scale: float | None = None, path: str | None = None):
        """Sample images for ``prompt_tokens[B, L]`` (ids into the stand-in encoder tables); needs
        the autoencoder.  Returns the images, and writes the first one to ``path`` when given."""
        from .sampling import generate_image, save_image

        if self.autoencoder is None:
            raise RuntimeError("image generation needs FluxTrainer.Config.autoencoder")
        tok = prompt_tokens.to(self.device)
        empty = torch.zeros_like(tok)
        img = generate_image(self.model, self.autoencoder, txt=self.t5_table[tok], vec=self.clip_table[tok[:, 0]],
                             img_height=self.config.img_size, img_width=self.config.img_size, steps=steps,
                             empty_txt=self.t5_table[empty] if guidance_scale is not None else None,
                             empty_vec=self.clip_table[empty[:, 0]] if guidance_scale is not None else None,
                             guidance_scale=guidance_scale, generator=self.gen)
        if path is not None:
            save_image(img, path)
        return img

    def train(self) -> None:
        t0 = time.time()
        for step in range(1, self.config.steps + 1):
            loss = self.train_step()
            self.losses.append(loss)
            if step % self.config.log_freq == 0:
                logger.info(f"flux step {step}: loss {loss:.4f} ({time.time() - t0:.1f}s)")

    def close(self) -> None:
        pass
