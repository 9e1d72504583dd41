"""Parameter and FLOP accounting shared by the model families.

FLOPs per token follow the reference's convention so MFU numbers are comparable:
dense ``6 * (N - N_embedding) + 6 * L * n_heads * (qk_dim + v_dim) * seq_len``
(causal sparsity not discounted, recomputation not counted); MoE counts the
shared experts plus ``top_k`` routed experts.  Parity: torchtitan/models/utils.py:412-545.
"""

from __future__ import annotations

import torch.nn as nn


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def count_params_and_flops(cfg, model: nn.Module | None, seq_len: int) -> tuple[int, float]:
    """Works from the *config* so that the answer is the global (unsharded) model size."""
    dim, vocab = cfg.dim, cfg.vocab_size
    emb = vocab * dim
    total = emb + dim  # embeddings + final norm
    if not cfg.enable_weight_tying:
        total += emb
    active = total
    attn_flops = 0.0
    for blk in list(cfg.layers) + list(getattr(cfg, "mtp_layers", None) or []):
        a = blk.attention
        n_attn, qk_dim, v_dim, heads = attention_params(a, dim)
        layer = n_attn + 2 * dim
        if hasattr(blk, "eh_proj"):   # multi-token prediction depth: three more norms and the fusion projection
            layer += 3 * dim + 2 * dim * dim
        if hasattr(blk, "post_attention_norm"):
            layer += 2 * dim
        layer_active = layer
        if blk.feed_forward is not None:
            f = 3 * dim * blk.feed_forward.hidden_dim
            layer += f
            layer_active += f
        if blk.moe is not None:
            m = blk.moe
            per_expert = 3 * dim * m.hidden_dim
            router = m.num_experts * dim
            if hasattr(m.routed_experts.inner_experts, "swiglu_limit"):  # biased experts (GPT-OSS)
                per_expert += 2 * m.hidden_dim + dim
            if getattr(m.router, "gate_bias", False):
                router += m.num_experts
            shared = 3 * dim * m.shared_hidden_dim if m.shared_hidden_dim else 0
            if shared and getattr(m, "shared_expert_gate", False):
                shared += dim                     # the sigmoid gate of the shared experts
            layer += m.num_experts * per_expert + router + shared
            layer_active += m.top_k * per_expert + router + shared
        total += layer
        active += layer_active
        attn_flops += 6 * heads * (qk_dim + v_dim) * seq_len
    vis = getattr(cfg, "vision_encoder", None)
    if vis is not None:     # vision tower: counted as parameters; its FLOPs depend on the images, not on seq_len
        d, mlp, dm = vis.dim, vis.mlp_dim, vis.dim * vis.spatial_merge ** 2
        n_blocks = len(vis.layers) or vis.n_layers
        v = vis.in_channels * getattr(vis, "temporal_patch_size", 1) * vis.patch_size ** 2 * d + d
        v += getattr(vis, "num_position_embeddings", 0) * d
        v += n_blocks * (3 * d * d + 3 * d + d * d + d + d * mlp + mlp + mlp * d + d + 4 * d)
        v += 2 * d + dm * dm + dm + dm * dim + dim
        total += v
    matmul_params = active if cfg.enable_weight_tying else active - emb
    return total, 6 * matmul_params + attn_flops


def attention_params(a, dim: int) -> tuple[int, int, int, int]:
    """``(param count, qk head dim, v head dim, n_heads)`` of an attention config."""
    if hasattr(a, "n_key_heads"):  # gated delta net: no softmax attention FLOPs (state updates are linear in T)
        kd, vd = a.n_key_heads * a.key_head_dim, a.n_value_heads * a.value_head_dim
        n = dim * (2 * kd + 2 * vd + 2 * a.n_value_heads) + (2 * kd + vd) * a.conv_kernel_size
        n += 2 * a.n_value_heads + a.value_head_dim + vd * dim
        return n, 0, 0, 0
    if hasattr(a, "kv_lora_rank"):  # multi-head latent attention
        h = a.n_heads
        qk = a.qk_nope_head_dim + a.qk_rope_head_dim
        n = 0
        if a.q_lora_rank:
            n += dim * a.q_lora_rank + a.q_lora_rank + a.q_lora_rank * h * qk
        else:
            n += dim * h * qk
        n += dim * (a.kv_lora_rank + a.qk_rope_head_dim) + a.kv_lora_rank
        n += a.kv_lora_rank * h * (a.qk_nope_head_dim + a.v_head_dim)
        n += h * a.v_head_dim * dim
        return n, qk, a.v_head_dim, h
    h = a.n_heads
    kv = a.n_kv_heads or h
    hd = a.head_dim or dim // h
    n = dim * (h + 2 * kv) * hd + h * hd * dim
    if getattr(a.wqkv, "bias", False):
        n += (h + 2 * kv) * hd
    if getattr(a.wo, "bias", False):
        n += dim
    if a.qk_norm is not None and getattr(a.qk_norm, "elementwise_affine", True):
        n += 2 * hd
    if getattr(a, "o_gate", None) is not None:
        n += dim * h * hd
    if getattr(a, "use_sinks", False):
        n += h
    return n, hd, hd, h
