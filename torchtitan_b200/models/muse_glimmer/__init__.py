"""Muse Glimmer family (text decoder): iRoPE (every fourth layer counted from the end has no
positional encoding), cyclic sliding-window / global attention pattern, gain-centred pre- and
post-norms, scale-free QK norm with a tuned query scale, sigmoid output gate, normalised token
embeddings and a multiplied, tanh-capped output head.  Hyper-parameters follow
torchtitan/models/muse_glimmer/__init__.py:60-520 (flavors debugmodel, 30B).  The vision encoder /
adapter of the multimodal flavors is not built here.
"""

from __future__ import annotations

import math

from torchtitan_b200.models.common.decoder import Decoder
from torchtitan_b200.models.common.layers import FeedForward, Linear, RMSNorm, RoPE
from torchtitan_b200.models.spec import ModelSpec

from .model import EmbeddingNorm, GainCenterRMSNorm, MuseAttention, MuseBlock

__all__ = ["muse_glimmer_configs", "model_registry", "build_muse_glimmer_config"]

_SCALE_QUERY_NUMERATOR = 43.7840518911
_NORM_EPS, _POST_NORM_EPS = 1e-5, 1e-8
_ROPE_THETA = 500_000.0
_EVERY_N_LAYERS_NOPE = 4
_FFN_DIM_MULTIPLIER = 3.0


def _use_rope(layer_id: int, n_layers: int) -> bool:
    return (n_layers - layer_id - 1) % _EVERY_N_LAYERS_NOPE != 0


def _window(layer_id: int, n_layers: int, pattern: list[int]) -> int | None:
    back = layer_id + _EVERY_N_LAYERS_NOPE - n_layers % _EVERY_N_LAYERS_NOPE
    w = pattern[back % len(pattern)]
    return w if w > 0 else None


def _gain(dim, eps, center):
    return GainCenterRMSNorm.Config(dim=dim, eps=eps, gain_center=center)


def build_muse_glimmer_config(*, dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, max_context_length,
                              window_pattern, output_multiplier) -> Decoder.Config:
    hidden = int(_FFN_DIM_MULTIPLIER * dim)
    layers = []
    for i in range(n_layers):
        depth_std = 0.02 / (2 * (i + 1)) ** 0.5
        attn = MuseAttention.Config(
            dim=dim, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
            wqkv=Linear.Config(init_std=0.02), wo=Linear.Config(init_std=depth_std),
            qk_norm=RMSNorm.Config(dim=head_dim, eps=_NORM_EPS, elementwise_affine=False),
            rope=RoPE.Config(dim=head_dim, theta=_ROPE_THETA, style="complex", max_context_length=max_context_length),
            use_rope=_use_rope(i, n_layers), scale_query_by=_SCALE_QUERY_NUMERATOR / math.sqrt(head_dim),
            o_gate=Linear.Config(init_std=0.02), sliding_window=_window(i, n_layers, window_pattern),
            softmax_scale=1.0 / math.sqrt(head_dim))
        ff = FeedForward.Config(dim=dim, hidden_dim=hidden, w13=Linear.Config(init_std=0.02),
                                w2=Linear.Config(init_std=depth_std))
        layers.append(MuseBlock.Config(
            layer_id=i, attention=attn, feed_forward=ff,
            attention_norm=_gain(dim, _NORM_EPS, 1.0), ffn_norm=_gain(dim, _NORM_EPS, 1.0),
            post_attention_norm=_gain(dim, _POST_NORM_EPS, 1.0), post_ffn_norm=_gain(dim, _POST_NORM_EPS, 1.0)))
    return Decoder.Config(
        dim=dim, vocab_size=vocab_size, n_layers=n_layers, layers=layers,
        tok_embeddings=EmbeddingNorm.Config(init_std=1.0, eps=_NORM_EPS),
        norm=_gain(dim, _NORM_EPS, 0.0),
        lm_head=Linear.Config(init_std=dim ** -0.5, init_cutoff=3.0),
        final_logit_softcap=20.0, final_logit_multiplier=output_multiplier,
        max_context_length=max_context_length)


def _mm(text_cfg, *, dim, heads, mlp, layers, patch, image_token_id):
    """Multimodal flavor: the shared ViT tower and adapter in front of the text decoder."""
    from torchtitan_b200.models.common.multimodal import to_multimodal
    from torchtitan_b200.models.common.vision_encoder import VisionEncoder

    vis = VisionEncoder.Config(patch_size=patch, dim=dim, num_heads=heads, mlp_dim=mlp, n_layers=layers, spatial_merge=2)
    return to_multimodal(text_cfg, vis, image_token_id)


muse_glimmer_configs = {
    "debugmodel": lambda: build_muse_glimmer_config(dim=256, n_layers=8, n_heads=4, n_kv_heads=2, head_dim=64,
                                                    vocab_size=2048, max_context_length=4096,
                                                    window_pattern=[128, 128, 128, 0], output_multiplier=1.0),
    "debugmodel_mm": lambda: _mm(muse_glimmer_configs["debugmodel"](), dim=64, heads=2, mlp=128, layers=2, patch=4,
                                 image_token_id=2047),
    "30B_mm": lambda: _mm(muse_glimmer_configs["30B"](), dim=1152, heads=16, mlp=4304, layers=27, patch=14,
                          image_token_id=202047),
    "30B": lambda: build_muse_glimmer_config(dim=6656, n_layers=52, n_heads=32, n_kv_heads=2, head_dim=128,
                                             vocab_size=202048, max_context_length=16384,
                                             window_pattern=[2048, 2048, 2048, 0], output_multiplier=0.19611613513),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in muse_glimmer_configs:
        raise ValueError(f"unknown muse_glimmer flavor '{flavor}' (have {sorted(muse_glimmer_configs)})")
    from torchtitan_b200.models.state_dict_adapter import StateDictAdapter
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.parallel.pipeline import pipeline_decoder

    return ModelSpec(name="muse_glimmer", flavor=flavor, model=muse_glimmer_configs[flavor](),
                     parallelize_fn=parallelize_decoder, pipelining_fn=pipeline_decoder, state_dict_adapter=StateDictAdapter)
