"""Images and videos for the multimodal pipeline: decode, fit to the vision tower's grid, normalise.

``fit_to_grid`` chooses an output size whose sides are multiples of ``patch_size * merge`` (the tower merges
``merge x merge`` patches into one token) and whose area lies inside a pixel budget, keeping the aspect ratio as
closely as the rounding allows.  ``load_image`` reads any format Pillow knows (or a saved ``.pt`` / ``.npy``
tensor); ``load_video`` decodes with OpenCV and keeps frames at a target rate between a minimum and a maximum
count, spread evenly over the clip.  ``process_image`` / ``process_video`` resize on uint8 (bicubic, antialiased),
scale to ``[0, 1]`` and normalise per channel, returning channel-first float tensors that the collator patchifies.

Parity: torchtitan/hf_datasets/multimodal/utils/image.py (smart_resize, image processing) and utils/video.py:19-148
(the reference decodes with PyAV; OpenCV is what this image provides).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from torchtitan_b200.utils.logging import logger

__all__ = ["fit_to_grid", "load_image", "process_image", "sample_frame_indices", "load_video", "process_video"]


def fit_to_grid(height: int, width: int, *, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    if min(height, width) <= 0:
        raise ValueError(f"empty image {height}x{width}")
    if max(height, width) / min(height, width) > 200:
        raise ValueError(f"aspect ratio {max(height, width) / min(height, width):.0f} is beyond 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:             # shrink both sides by the same ratio, rounding down
        s = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / s / factor) * factor)
        w = max(factor, math.floor(width / s / factor) * factor)
    elif h * w < min_pixels:           # grow, rounding up
        s = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * s / factor) * factor
        w = math.ceil(width * s / factor) * factor
    return h, w


def load_image(path: str) -> torch.Tensor:
    """``[C, H, W]`` uint8 (RGB) for image files; saved tensors are returned as they are."""
    if path.endswith(".pt"):
        return torch.load(path)
    if path.endswith(".npy"):
        import numpy as np

        return torch.from_numpy(np.load(path))
    import numpy as np
    from PIL import Image

    with Image.open(path) as im:
        return torch.from_numpy(np.asarray(im.convert("RGB")).copy()).permute(2, 0, 1)


def _resize_normalize(x: torch.Tensor, size: tuple[int, int], mean, std) -> torch.Tensor:
    """``[N, C, H, W]`` uint8 or float -> float32, resized and normalised."""
    is_u8 = x.dtype == torch.uint8
    y = F.interpolate(x.float(), size=size, mode="bicubic", align_corners=False, antialias=True)
    if is_u8:
        y = y.clamp_(0, 255) / 255.0
    m = torch.tensor(mean, dtype=torch.float32).view(1, -1, 1, 1)
    s = torch.tensor(std, dtype=torch.float32).view(1, -1, 1, 1)
    return (y - m) / s


def process_image(image: torch.Tensor, *, patch_size: int, merge_size: int, min_pixels: int = 56 * 56,
                  max_pixels: int = 1024 * 1024, image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5)) -> torch.Tensor:
    """``[C, H, W]`` -> ``[C, H', W']`` float32 with ``H'``, ``W'`` multiples of ``patch_size * merge_size``."""
    _, H, W = image.shape
    size = fit_to_grid(H, W, factor=patch_size * merge_size, min_pixels=min_pixels, max_pixels=max_pixels)
    return _resize_normalize(image[None], size, image_mean, image_std)[0]


def sample_frame_indices(total_frames: int, video_fps: float, *, fps: float = 2.0, min_frames: int = 4,
                         max_frames: int = 768) -> list[int]:
    """Evenly spaced frame indices: ``duration * fps`` of them, clamped to ``[min_frames, max_frames]`` and to the
    number of frames there are."""
    if total_frames <= 0:
        return []
    want = int(total_frames / max(video_fps, 1e-6) * fps)
    n = min(max(min_frames, min(want, max_frames)), total_frames)
    if n == 1:
        return [0]
    return [round(i * (total_frames - 1) / (n - 1)) for i in range(n)]


def load_video(path: str, *, fps: float = 2.0, min_frames: int = 4, max_frames: int = 768) -> torch.Tensor | None:
    """``[T, H, W, C]`` uint8 (RGB) of the sampled frames, or None when the file cannot be decoded.  Frames are
    decoded in order (inter-frame codecs need that) and only the sampled ones are kept."""
    try:
        import cv2
        import numpy as np

        cap = cv2.VideoCapture(path)
        if not cap.isOpened():
            raise OSError("cannot open")
        rate = float(cap.get(cv2.CAP_PROP_FPS) or 24.0)
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT) or 0)
        frames = []
        if total > 0:
            keep = set(sample_frame_indices(total, rate, fps=fps, min_frames=min_frames, max_frames=max_frames))
            i = 0
            while True:
                ok = cap.grab()
                if not ok:
                    break
                if i in keep:
                    ok, frame = cap.retrieve()
                    if ok:
                        frames.append(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB))
                i += 1
        else:                            # no frame count in the container: decode everything, then sample
            every = []
            while True:
                ok, frame = cap.read()
                if not ok:
                    break
                every.append(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB))
            frames = [every[i] for i in sample_frame_indices(len(every), rate, fps=fps, min_frames=min_frames,
                                                             max_frames=max_frames)]
        cap.release()
        if not frames:
            return None
        return torch.from_numpy(np.stack(frames))
    except Exception as e:
        logger.warning(f"could not load video {path}: {e}")
        return None


def process_video(video: torch.Tensor, *, patch_size: int, merge_size: int, min_pixels: int = 56 * 56,
                  max_pixels: int = 512 * 512, image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5)) -> torch.Tensor:
    """``[T, H, W, C]`` uint8 -> ``[T, C, H', W']`` float32; the pixel budget is per frame."""
    _, H, W, _ = video.shape
    size = fit_to_grid(H, W, factor=patch_size * merge_size, min_pixels=min_pixels, max_pixels=max_pixels)
    return _resize_normalize(video.permute(0, 3, 1, 2), size, image_mean, image_std)
