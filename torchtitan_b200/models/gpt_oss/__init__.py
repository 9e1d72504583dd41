"""GPT-OSS family (20B, 120B): grouped-query attention with learned attention sinks and biases,
sliding-window attention on every other layer, YaRN RoPE, MoE in every layer with biased experts
and a clamped SwiGLU.  Hyper-parameters follow torchtitan/models/gpt_oss/__init__.py and
model.py:34-273.
"""

from __future__ import annotations

from torchtitan_b200.models.common.attention import GQAttention
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.layers import Embedding, Linear, RMSNorm, RoPE
from torchtitan_b200.models.common.moe import MoE, RoutedExperts, TokenChoiceTopKRouter
from torchtitan_b200.models.spec import ModelSpec

from .moe import GptOssExperts

__all__ = ["gpt_oss_configs", "model_registry", "build_gpt_oss_config"]

_EPS = 1e-5


def build_gpt_oss_config(*, dim, n_layers, n_heads=64, n_kv_heads=8, head_dim=64, moe_hidden_dim=2880, num_experts=32,
                         top_k=4, vocab_size=201088, sliding_window=128, rope_theta=150000.0, rope_factor=32.0,
                         original_seq_len=4096, max_context_length=4096) -> Decoder.Config:
    out_std = 0.02 / (2 * n_layers) ** 0.5
    # YaRN's attention magnitude correction m = 0.1 ln(factor) + 1 scales q and k alike: it is folded into the softmax
    # scale as m^2, the rotary table stays a pure rotation (parity: torchtitan/models/gpt_oss/model.py:74-78)
    import math

    mscale = 0.1 * math.log(rope_factor) + 1.0 if rope_factor > 1.0 else 1.0
    softmax_scale = head_dim ** -0.5 * mscale * mscale
    layers = []
    for i in range(n_layers):
        attn = GQAttention.Config(
            dim=dim, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, softmax_scale=softmax_scale,
            wqkv=Linear.Config(init_std=0.02, bias=True), wo=Linear.Config(init_std=out_std, bias=True),
            rope=RoPE.Config(dim=head_dim, theta=rope_theta, style="cos_sin", scaling="yarn", rope_factor=rope_factor,
                             beta_fast=32.0, beta_slow=1.0, original_seq_len=original_seq_len, truncate=False,
                             max_context_length=max_context_length),
            sliding_window=sliding_window if i % 2 == 0 else None, use_sinks=True)
        moe = MoE.Config(
            dim=dim, hidden_dim=moe_hidden_dim, num_experts=num_experts, top_k=top_k,
            router=TokenChoiceTopKRouter.Config(score_func="softmax", route_norm=True, route_scale=1.0, gate_bias=True),
            routed_experts=RoutedExperts.Config(inner_experts=GptOssExperts.Config(init_std=0.02, out_init_std=out_std)),
            load_balance_coeff=1e-3)
        layers.append(TransformerBlock.Config(layer_id=i, attention=attn, moe=moe,
                                              attention_norm=RMSNorm.Config(dim=dim, eps=_EPS),
                                              ffn_norm=RMSNorm.Config(dim=dim, eps=_EPS)))
    return Decoder.Config(dim=dim, vocab_size=vocab_size, n_layers=n_layers, layers=layers,
                          tok_embeddings=Embedding.Config(init_std=1.0), norm=RMSNorm.Config(dim=dim, eps=_EPS),
                          lm_head=Linear.Config(init_std=dim ** -0.5, init_cutoff=3.0),
                          max_context_length=max_context_length)


gpt_oss_configs = {
    "debugmodel": lambda: build_gpt_oss_config(dim=256, n_layers=4, n_heads=8, n_kv_heads=4, head_dim=32, moe_hidden_dim=256,
                                               num_experts=8, top_k=4, vocab_size=2048, sliding_window=64),
    "20B": lambda: build_gpt_oss_config(dim=2880, n_layers=24, num_experts=32),
    "120B": lambda: build_gpt_oss_config(dim=2880, n_layers=36, num_experts=128),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in gpt_oss_configs:
        raise ValueError(f"unknown gpt_oss flavor '{flavor}' (have {sorted(gpt_oss_configs)})")
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.parallel.pipeline import pipeline_decoder

    from .state_dict_adapter import GptOssStateDictAdapter

    return ModelSpec(name="gpt_oss", flavor=flavor, model=gpt_oss_configs[flavor](), parallelize_fn=parallelize_decoder,
                     pipelining_fn=pipeline_decoder, state_dict_adapter=GptOssStateDictAdapter)
