"""Swap the mixture-of-experts blocks of a Hugging Face model for this framework's ``MoE`` layer.

The HF blocks loop over experts in Python; the native layer routes with the fused router, permutes token slots into
padded expert-major order and runs grouped GEMMs (and can be put under expert parallelism like any native MoE).
``swap_native_moe`` walks the decoder layers, recognises the block family from its attributes, builds a native
layer of the same shape, copies the weights and installs an adapter with the HF block's calling convention
(``[batch, seq, dim]`` in and out).

Recognised layouts (``transformers`` 5.x, experts stored as 3-D ``gate_up_proj [E, 2F, D]`` / ``down_proj [E, D, F]``):

* softmax top-k router with optional renormalisation (Qwen3-MoE and its relatives): ``block.gate`` holds
  ``weight``, ``top_k``, ``norm_topk_prob``;
* sigmoid router with expert groups, a selection bias, a scaling factor and always-on shared experts
  (DeepSeek-V3 and its relatives): ``block.gate`` holds ``weight`` and ``e_score_correction_bias``, the block
  ``n_group`` / ``topk_group`` / ``routed_scaling_factor`` / ``shared_experts``.

``restore_hf_moe_state`` writes trained native weights back into HF tensors, so ``save_pretrained`` of the swapped
model's original blocks still works for export.

Parity: torchtitan/experiments/transformers_modeling_backend/moe_replacement.py:49-587.
"""

from __future__ import annotations

import torch
import torch.nn as nn

__all__ = ["probe_hf_moe_block", "build_native_moe", "NativeMoEAdapter", "swap_native_moe", "restore_hf_moe_state"]


def _moe_attr(layer: nn.Module) -> str | None:
    """Name of the decoder layer's attribute that holds an MoE block (``mlp`` or ``block_sparse_moe``)."""
    for name in ("mlp", "block_sparse_moe", "feed_forward"):
        blk = getattr(layer, name, None)
        if blk is not None and hasattr(blk, "experts") and hasattr(blk, "gate"):
            return name
    return None


def probe_hf_moe_block(block: nn.Module) -> dict:
    """Shape and routing parameters of one HF MoE block; raises ``NotImplementedError`` for unknown layouts."""
    ex, gate = block.experts, block.gate
    if not (hasattr(ex, "gate_up_proj") and hasattr(ex, "down_proj") and ex.gate_up_proj.dim() == 3):
        raise NotImplementedError(f"{type(block).__name__}: experts are not stored as gate_up_proj / down_proj 3-D tensors")
    if getattr(ex, "gate_up_proj_bias", None) is not None:
        raise NotImplementedError(f"{type(block).__name__}: biased experts are not covered")
    E, F2, D = ex.gate_up_proj.shape
    info = dict(num_experts=E, hidden_dim=F2 // 2, dim=D, shared_hidden_dim=0, route_scale=1.0, groups=None,
                limited_groups=None, bias=None)
    if hasattr(gate, "e_score_correction_bias"):
        info.update(score_func="sigmoid", top_k=int(block.top_k), route_norm=bool(block.norm_topk_prob),
                    route_scale=float(block.routed_scaling_factor), groups=int(block.n_group),
                    limited_groups=int(block.topk_group), bias=gate.e_score_correction_bias)
        shared = getattr(block, "shared_experts", None)
        if shared is not None:
            info["shared_hidden_dim"] = shared.gate_proj.weight.shape[0]
    elif hasattr(gate, "top_k") and hasattr(gate, "weight"):
        info.update(score_func="softmax", top_k=int(gate.top_k), route_norm=bool(getattr(gate, "norm_topk_prob", False)))
    else:
        raise NotImplementedError(f"{type(gate).__name__}: unknown router layout")
    return info


def build_native_moe(block: nn.Module, *, dtype=None, device=None):
    """A native ``MoE`` with the block's shape and weights."""
    from torchtitan_b200.models.common.layers import FeedForward
    from torchtitan_b200.models.common.moe import MoE, TokenChoiceTopKRouter

    p = probe_hf_moe_block(block)
    cfg = MoE.Config(
        dim=p["dim"], hidden_dim=p["hidden_dim"], num_experts=p["num_experts"], top_k=p["top_k"],
        router=TokenChoiceTopKRouter.Config(score_func=p["score_func"], route_norm=p["route_norm"],
                                            route_scale=p["route_scale"], num_expert_groups=p["groups"],
                                            num_limited_groups=p["limited_groups"]),
        load_balance_coeff=1e-3 if p["bias"] is not None else None, shared_hidden_dim=p["shared_hidden_dim"],
        shared_experts=FeedForward.Config() if p["shared_hidden_dim"] else None)
    ref = block.experts.gate_up_proj
    moe = cfg.build().to(device=device or ref.device, dtype=dtype or ref.dtype)
    moe.init_buffers(device or ref.device)
    F = p["hidden_dim"]
    ie = moe.routed_experts.inner_experts
    with torch.no_grad():
        ie.w1_EFD.copy_(block.experts.gate_up_proj[:, :F])
        ie.w3_EFD.copy_(block.experts.gate_up_proj[:, F:])
        ie.w2_EDF.copy_(block.experts.down_proj)
        moe.router.gate.weight.copy_(block.gate.weight)
        if p["bias"] is not None:
            moe.expert_bias_E.copy_(p["bias"].float())
        if p["shared_hidden_dim"]:
            sh = block.shared_experts
            moe.shared_experts.w13.weight.copy_(torch.cat([sh.gate_proj.weight, sh.up_proj.weight]))
            moe.shared_experts.w2.weight.copy_(sh.down_proj.weight)
    return moe


class NativeMoEAdapter(nn.Module):
    """The native layer behind the HF block's interface; keeps the replaced block (without registering it as a
    submodule, so its parameters are neither trained nor sharded) for ``restore_hf_moe_state``."""

    def __init__(self, moe: nn.Module, original: nn.Module):
        super().__init__()
        self.moe = moe
        object.__setattr__(self, "_original", original)

    def forward(self, hidden_states: torch.Tensor, *_, **__) -> torch.Tensor:
        shape = hidden_states.shape
        return self.moe(hidden_states.reshape(-1, shape[-1])).reshape(shape)


def _decoder_layers(model) -> list[nn.Module]:
    hf = getattr(model, "hf", model)
    return list(hf.model.layers)


def swap_native_moe(model, *, dtype=None) -> int:
    """Replace every recognised MoE block; returns how many were replaced (dense layers are left alone)."""
    n = 0
    for layer in _decoder_layers(model):
        name = _moe_attr(layer)
        if name is None or isinstance(getattr(layer, name), NativeMoEAdapter):
            continue
        block = getattr(layer, name)
        setattr(layer, name, NativeMoEAdapter(build_native_moe(block, dtype=dtype), block))
        n += 1
    return n


@torch.no_grad()
def restore_hf_moe_state(model) -> int:
    """Copy the native layers' weights back into the HF blocks they replaced and put those blocks back."""
    n = 0
    for layer in _decoder_layers(model):
        for name in ("mlp", "block_sparse_moe", "feed_forward"):
            ad = getattr(layer, name, None)
            if not isinstance(ad, NativeMoEAdapter):
                continue
            blk, moe = ad._original, ad.moe
            ie = moe.routed_experts.inner_experts
            blk.experts.gate_up_proj.copy_(torch.cat([ie.w1_EFD, ie.w3_EFD], dim=1))
            blk.experts.down_proj.copy_(ie.w2_EDF)
            blk.gate.weight.copy_(moe.router.gate.weight)
            if hasattr(blk.gate, "e_score_correction_bias") and moe.expert_bias_E is not None:
                blk.gate.e_score_correction_bias.copy_(moe.expert_bias_E)
            if moe.shared_experts is not None:
                F = moe.shared_experts.w13.weight.shape[0] // 2
                blk.shared_experts.gate_proj.weight.copy_(moe.shared_experts.w13.weight[:F])
                blk.shared_experts.up_proj.weight.copy_(moe.shared_experts.w13.weight[F:])
                blk.shared_experts.down_proj.weight.copy_(moe.shared_experts.w2.weight)
            setattr(layer, name, blk)
            n += 1
    return n
