"""Multimodal batches: interleaved text and images as one packed token stream plus packed patches.

A sample is a list of segments, text (token ids) or image (``[C, H, W]`` float tensor).  The
collator turns each image into ``gh x gw`` patches of ``patch_size`` (height and width are cropped
to multiples of ``patch_size * merge``), emits ``gh * gw / merge^2`` placeholder tokens for it
(labels ignored), packs samples into the batch's ``num_tokens_per_batch`` tokens with positions
restarting per sample, and pads with one ignored tail document.  A sample that does not fit in
what is left of the batch is carried to the next one; images are never cut.

Batch: ``({"input", "positions", "pixel_patches" [N, C p p], "grid_hw" [I, 2]}, labels)``.

``dataset = "synthetic_mm"`` draws random text and images, a pure function of
``(seed, dp rank, batch index)``.  ``dataset = "mm_jsonl"`` reads lines
``{"segments": [{"text": ...} | {"image": "<.png / .jpg / ... or a .pt / .npy tensor>"} | {"video": "<file>",
"fps": 2.0, "max_frames": 32}]}`` (``components/data/media.py`` decodes, resizes to the patch grid and normalises).
Parity: torchtitan/hf_datasets/multimodal/mm_datasets.py and mm_collator.py (interleaved
samples, patchification, placeholder expansion, padding to the batch length).
"""

from __future__ import annotations

import json
from typing import Any, Iterator

import torch

from torchtitan_b200.ops.reference import IGNORE_INDEX

from . import media
from .loader import BaseDataLoader

__all__ = ["patchify", "MultimodalCollator", "MultimodalDataLoader"]


def patchify(image: torch.Tensor, patch: int, merge: int) -> tuple[torch.Tensor, tuple[int, int]]:
    """``[C, H, W]`` -> ``(patches [gh * gw, C * patch * patch], (gh, gw))``, row-major over the grid."""
    C, H, W = image.shape
    q = patch * merge
    gh, gw = (H // q) * merge, (W // q) * merge
    if gh == 0 or gw == 0:
        raise ValueError(f"image {H}x{W} is smaller than one merged patch ({q}x{q})")
    x = image[:, : gh * patch, : gw * patch].reshape(C, gh, patch, gw, patch)
    return x.permute(1, 3, 0, 2, 4).reshape(gh * gw, C * patch * patch).contiguous(), (gh, gw)


class MultimodalCollator:
    def __init__(self, num_tokens: int, patch: int, merge: int, image_token_id: int, max_context_length: int):
        self.T, self.patch, self.merge, self.img_id = num_tokens, patch, merge, image_token_id
        self.ctx = min(max_context_length, num_tokens)

    def encode(self, segments: list) -> tuple[list[int], list[int], list[torch.Tensor], list[tuple[int, int]]]:
        """One sample -> (inputs, labels, patch tensors, grids); next-token labels, image slots ignored."""
        ids: list[int] = []
        is_img: list[bool] = []
        patches, grids = [], []
        for seg in segments:
            if isinstance(seg, torch.Tensor):
                p, (gh, gw) = patchify(seg, self.patch, self.merge)
                n = gh * gw // (self.merge ** 2)
                ids += [self.img_id] * n
                is_img += [True] * n
                patches.append(p)
                grids.append((gh, gw))
            else:
                ids += list(seg)
                is_img += [False] * len(seg)
        inp = ids[:-1]
        lab = [IGNORE_INDEX if is_img[i + 1] else ids[i + 1] for i in range(len(ids) - 1)]
        return inp, lab, patches, grids

    def collate(self, samples: list[tuple]) -> tuple[dict[str, torch.Tensor], torch.Tensor]:
        T = self.T
        inp = torch.zeros(T, dtype=torch.int64)
        lab = torch.full((T,), IGNORE_INDEX, dtype=torch.int64)
        pos = torch.zeros(T, dtype=torch.int64)
        o = 0
        patches, grids = [], []
        for a, b, p, g in samples:
            n = len(a)
            inp[o:o + n] = torch.tensor(a, dtype=torch.int64)
            lab[o:o + n] = torch.tensor(b, dtype=torch.int64)
            pos[o:o + n] = torch.arange(n)
            o += n
            patches += p
            grids += g
        if o < T:
            pos[o:] = torch.arange(T - o)
        c = patches[0].shape[1] if patches else 0
        return ({"input": inp, "positions": pos,
                 "pixel_patches": torch.cat(patches) if patches else torch.zeros(0, c),
                 "grid_hw": torch.tensor(grids, dtype=torch.int64).reshape(-1, 2)}, lab)


class MultimodalDataLoader(BaseDataLoader):
    def __init__(self, config: BaseDataLoader.Config, *, dp_world_size: int = 1, dp_rank: int = 0,
                 num_tokens_per_batch: int = 2048, max_context_length: int = 2048, vocab_size: int = 2048,
                 tokenizer=None, patch_size: int = 14, spatial_merge: int = 2, image_token_id: int = 0,
                 in_channels: int = 3, **_):
        self.config = config
        self.dp_world_size, self.dp_rank = dp_world_size, dp_rank
        self.collator = MultimodalCollator(num_tokens_per_batch, patch_size, spatial_merge, image_token_id, max_context_length)
        self.vocab = (config.synthetic_vocab_size or vocab_size)
        self.img_id, self.channels = image_token_id, in_channels
        self.tokenizer = tokenizer
        self.batch_idx = 0
        self.cursor = 0
        self.carry: tuple | None = None
        self.lines: list[str] | None = None
        if config.dataset == "mm_jsonl":
            if not config.dataset_path:
                raise ValueError("dataset 'mm_jsonl' needs dataloader.dataset_path")
            with open(config.dataset_path) as f:
                lines = [ln for ln in f if ln.strip()]
            self.lines = lines[dp_rank::dp_world_size]
            if not self.lines:
                raise ValueError("the multimodal dataset has fewer samples than dp ranks")

    # -- sample streams ---------------------------------------------------------------------
    def _synthetic_sample(self, g: torch.Generator) -> list:
        q = self.collator.patch * self.collator.merge
        segs: list = []
        n_txt = int(torch.randint(8, 48, (1,), generator=g))
        txt = torch.randint(0, self.vocab, (n_txt,), generator=g)
        txt[txt == self.img_id] = (self.img_id + 1) % self.vocab
        segs.append(txt.tolist())
        if torch.rand(1, generator=g).item() < 0.7:
            h, w = (int(v) for v in torch.randint(1, 4, (2,), generator=g))
            segs.append(torch.randn(self.channels, h * q, w * q, generator=g))
            tail = torch.randint(0, self.vocab, (int(torch.randint(4, 24, (1,), generator=g)),), generator=g)
            tail[tail == self.img_id] = (self.img_id + 1) % self.vocab
            segs.append(tail.tolist())
        return segs

    def _jsonl_sample(self) -> list:
        rec = json.loads(self.lines[self.cursor % len(self.lines)])
        self.cursor += 1
        segs: list = []
        for s in rec["segments"]:
            if "image" in s:
                segs.append(self._image(media.load_image(s["image"])))
            elif "video" in s:
                # every sampled frame becomes one image segment (its own patch grid); a tower with temporal patches
                # repeats a single frame over the temporal extent, as for still images
                clip = media.load_video(s["video"], fps=s.get("fps", 2.0), min_frames=s.get("min_frames", 4),
                                        max_frames=s.get("max_frames", 32))
                if clip is None:
                    continue
                q = self.collator.patch
                frames = media.process_video(clip, patch_size=q, merge_size=self.collator.merge,
                                             max_pixels=s.get("max_pixels", 256 * 256))
                segs += list(frames)
            else:
                if self.tokenizer is None:
                    raise ValueError("text segments need a tokenizer")
                segs.append(self.tokenizer.encode(s["text"], add_bos=not segs, add_eos=False))
        return segs

    def _image(self, image: torch.Tensor) -> torch.Tensor:
        """Saved float tensors are taken as already prepared; decoded (uint8) images are fitted to the patch grid
        and normalised."""
        if image.dtype != torch.uint8:
            return image.float()
        return media.process_image(image, patch_size=self.collator.patch, merge_size=self.collator.merge)

    def _make(self, idx: int):
        g = torch.Generator()
        g.manual_seed((self.config.seed * 1_000_003 + self.dp_rank) * 1_000_003 + idx)
        T = self.collator.T
        chosen, fill = [], 0
        if self.carry is not None:
            chosen.append(self.carry)
            fill = len(self.carry[0])
            self.carry = None
        while True:
            enc = self.collator.encode(self._jsonl_sample() if self.lines is not None else self._synthetic_sample(g))
            n = len(enc[0])
            if n > min(T, self.collator.ctx):
                continue            # a sample longer than the context is dropped (images are never cut)
            if fill + n > T:
                if self.lines is not None:
                    self.carry = enc
                break
            chosen.append(enc)
            fill += n
        return self.collator.collate(chosen)

    def __iter__(self) -> Iterator:
        while True:
            batch = self._make(self.batch_idx)
            self.batch_idx += 1
            yield batch

    def state_dict(self) -> dict[str, Any]:
        return {"version": 1, "dp_world_size": self.dp_world_size,
                f"dp_rank_{self.dp_rank}": {"batch_idx": self.batch_idx, "cursor": self.cursor}}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if not sd:
            return
        if sd.get("dp_world_size", self.dp_world_size) != self.dp_world_size:
            raise ValueError(f"dataloader state was saved with dp degree {sd.get('dp_world_size')}, cannot resume with "
                             f"{self.dp_world_size}")
        st = sd.get(f"dp_rank_{self.dp_rank}")
        if st:
            self.batch_idx, self.cursor = int(st["batch_idx"]), int(st.get("cursor", 0))
