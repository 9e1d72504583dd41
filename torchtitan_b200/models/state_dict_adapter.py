"""Native checkpoint names <-> Hugging Face names.

A family adapter declares ``hf_to_native`` (templates with ``{}`` for the layer
index and, for MoE, the expert index) and optional per-key tensor transforms.
``to_hf`` / ``from_hf`` operate on flat ``{name: tensor}`` dicts whose native side
uses the un-fused checkpoint names (``qkv_linear.wq`` ...).
Parity: torchtitan/protocols/state_dict_adapter.py:19-133.
"""

from __future__ import annotations

import json
import os
import re
from typing import Any, Callable

import torch

__all__ = ["StateDictAdapter", "pairs_to_halves", "halves_to_pairs"]


def pairs_to_halves(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Reorder each head's rows from adjacent-pair RoPE order ``(0,1),(2,3)..`` to
    rotate-half order ``0,2,4,..,1,3,5,..`` (the order Hugging Face Llama stores)."""
    rows = w.shape[0]
    hd = rows // n_heads
    idx = torch.arange(hd).view(hd // 2, 2).t().reshape(-1)  # 0,2,4..,1,3,5..
    full = (torch.arange(n_heads)[:, None] * hd + idx[None, :]).reshape(-1)
    return w.index_select(0, full.to(w.device))


def halves_to_pairs(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    rows = w.shape[0]
    hd = rows // n_heads
    idx = torch.arange(hd).view(2, hd // 2).t().reshape(-1)  # 0,hd/2,1,hd/2+1,..
    full = (torch.arange(n_heads)[:, None] * hd + idx[None, :]).reshape(-1)
    return w.index_select(0, full.to(w.device))


class StateDictAdapter:
    hf_to_native: dict[str, str | None] = {}

    def __init__(self, model_config, hf_assets_path: str | None = None):
        self.model_config = model_config
        self.hf_assets_path = hf_assets_path
        self.fqn_to_index_mapping: dict[str, int] | None = None
        if hf_assets_path:
            idx = os.path.join(hf_assets_path, "model.safetensors.index.json")
            if os.path.exists(idx):
                with open(idx) as f:
                    weight_map = json.load(f).get("weight_map", {})
                self.fqn_to_index_mapping = {
                    k: int(re.search(r"(\d+)-of-", v).group(1)) if re.search(r"(\d+)-of-", v) else 1
                    for k, v in weight_map.items()
                }
        self._native_to_hf = {v: k for k, v in self.hf_to_native.items() if v is not None}

    # -- hooks for subclasses ---------------------------------------------
    def transform_to_hf(self, native_key: str, tensor: torch.Tensor) -> torch.Tensor:
        return tensor

    def transform_from_hf(self, native_key: str, tensor: torch.Tensor) -> torch.Tensor:
        return tensor

    # -- generic translation ----------------------------------------------
    @staticmethod
    def _abstract(key: str) -> tuple[str, list[str]]:
        nums = re.findall(r"(?<=\.)\d+(?=\.)", key)
        return re.sub(r"(?<=\.)\d+(?=\.)", "{}", key), nums

    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        out = {}
        for key, val in state_dict.items():
            templ, nums = self._abstract(key)
            if templ not in self._native_to_hf:
                raise KeyError(f"no Hugging Face name for '{key}'")
            out[self._native_to_hf[templ].format(*nums)] = self.transform_to_hf(templ, val)
        return out

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out = {}
        for key, val in hf_state_dict.items():
            templ, nums = self._abstract(key)
            if templ not in self.hf_to_native:
                raise KeyError(f"unexpected Hugging Face key '{key}'")
            native = self.hf_to_native[templ]
            if native is None:
                continue
            out[native.format(*nums)] = self.transform_from_hf(native, val)
        return out

    def get_hf_storage_reader(self, path: str):
        from torch.distributed.checkpoint import HuggingFaceStorageReader

        return HuggingFaceStorageReader(path)
