"""Qwen3 family: dense 0.6B-32B and MoE (30B-A3B, 235B-A22B).

QK-RMSNorm (eps 1e-6), rotate-half RoPE with theta 1e6, softmax router with renormalised
top-k weights, residual-output init ``0.02 / sqrt(2 * n_layers)``.  Hyper-parameters follow
torchtitan/models/qwen3/__init__.py:52-635.
"""

from __future__ import annotations

from torchtitan_b200.models.common.attention import GQAttention
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.layers import Embedding, FeedForward, Linear, RMSNorm, RoPE
from torchtitan_b200.models.common.moe import GroupedExperts, MoE, RoutedExperts, TokenChoiceTopKRouter
from torchtitan_b200.models.spec import ModelSpec

__all__ = ["qwen3_configs", "model_registry", "build_qwen3_config"]

_EPS = 1e-6


def build_qwen3_config(*, dim, n_layers, n_heads, n_kv_heads, head_dim=128, hidden_dim=0, vocab_size=151936,
                       weight_tying=False, max_context_length=4096, rope_theta=1e6, moe_hidden_dim=0,
                       num_experts=0, top_k=0, embed_std=0.02) -> Decoder.Config:
    out_std = 0.02 / (2 * n_layers) ** 0.5
    layers = []
    for i in range(n_layers):
        attn = GQAttention.Config(
            dim=dim, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
            wqkv=Linear.Config(init_std=0.02), wo=Linear.Config(init_std=out_std),
            qk_norm=RMSNorm.Config(dim=head_dim, eps=_EPS),
            rope=RoPE.Config(dim=head_dim, theta=rope_theta, style="cos_sin", max_context_length=max_context_length))
        ff = moe = None
        if num_experts:
            moe = MoE.Config(
                dim=dim, hidden_dim=moe_hidden_dim, num_experts=num_experts, top_k=top_k,
                router=TokenChoiceTopKRouter.Config(score_func="softmax", route_norm=True, route_scale=1.0),
                routed_experts=RoutedExperts.Config(inner_experts=GroupedExperts.Config(init_std=0.02, out_init_std=out_std)),
                load_balance_coeff=1e-3)
        else:
            ff = FeedForward.Config(dim=dim, hidden_dim=hidden_dim, w13=Linear.Config(init_std=0.02),
                                    w2=Linear.Config(init_std=out_std))
        layers.append(TransformerBlock.Config(layer_id=i, attention=attn, feed_forward=ff, moe=moe,
                                              attention_norm=RMSNorm.Config(dim=dim, eps=_EPS),
                                              ffn_norm=RMSNorm.Config(dim=dim, eps=_EPS)))
    return Decoder.Config(dim=dim, vocab_size=vocab_size, n_layers=n_layers, layers=layers,
                          tok_embeddings=Embedding.Config(init_std=embed_std), norm=RMSNorm.Config(dim=dim, eps=_EPS),
                          lm_head=Linear.Config(init_std=dim ** -0.5, init_cutoff=3.0),
                          enable_weight_tying=weight_tying, max_context_length=max_context_length)


qwen3_configs = {
    "debugmodel": lambda: build_qwen3_config(dim=256, n_layers=8, n_heads=16, n_kv_heads=8, hidden_dim=3072,
                                             vocab_size=2048, weight_tying=True),
    "0.6B": lambda: build_qwen3_config(dim=1024, n_layers=28, n_heads=16, n_kv_heads=8, hidden_dim=3072, weight_tying=True),
    "1.7B": lambda: build_qwen3_config(dim=2048, n_layers=28, n_heads=16, n_kv_heads=8, hidden_dim=6144, weight_tying=True),
    "4B": lambda: build_qwen3_config(dim=2560, n_layers=36, n_heads=32, n_kv_heads=8, hidden_dim=9728, weight_tying=True),
    "8B": lambda: build_qwen3_config(dim=4096, n_layers=36, n_heads=32, n_kv_heads=8, hidden_dim=12288),
    "14B": lambda: build_qwen3_config(dim=5120, n_layers=40, n_heads=40, n_kv_heads=8, hidden_dim=17408),
    "32B": lambda: build_qwen3_config(dim=5120, n_layers=64, n_heads=64, n_kv_heads=8, hidden_dim=25600),
    "debugmodel_moe": lambda: build_qwen3_config(dim=256, n_layers=8, n_heads=16, n_kv_heads=8, vocab_size=2048,
                                                 moe_hidden_dim=768, num_experts=64, top_k=8),
    "debugmodel_moe_tiny": lambda: build_qwen3_config(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16, vocab_size=512,
                                                      moe_hidden_dim=32, num_experts=8, top_k=2, max_context_length=256),
    "30B-A3B": lambda: build_qwen3_config(dim=2048, n_layers=48, n_heads=32, n_kv_heads=4, moe_hidden_dim=768,
                                          num_experts=128, top_k=8, max_context_length=4096),
    "235B-A22B": lambda: build_qwen3_config(dim=4096, n_layers=94, n_heads=64, n_kv_heads=4, moe_hidden_dim=1536,
                                            num_experts=128, top_k=8),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in qwen3_configs:
        raise ValueError(f"unknown qwen3 flavor '{flavor}' (have {sorted(qwen3_configs)})")
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.parallel.pipeline import pipeline_decoder

    from .state_dict_adapter import Qwen3StateDictAdapter

    return ModelSpec(name="qwen3", flavor=flavor, model=qwen3_configs[flavor](), parallelize_fn=parallelize_decoder,
                     pipelining_fn=pipeline_decoder, state_dict_adapter=Qwen3StateDictAdapter)
