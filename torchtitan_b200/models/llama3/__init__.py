"""Llama 3.x family.

Flavors and hyper-parameters follow torchtitan/models/llama3/__init__.py:95-366;
initialisation follows :45-66 there (embeddings N(0,1), block linears truncated
normal std 0.02, residual-output projections depth-scaled ``0.02/sqrt(2(l+1))``,
``lm_head`` truncated at 3 sigma with std ``dim**-0.5``).
"""

from __future__ import annotations

import math

from torchtitan_b200.models.common.attention import GQAttention
from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.layers import Embedding, FeedForward, Linear, RMSNorm, RoPE, ffn_hidden_dim
from torchtitan_b200.models.spec import ModelSpec

__all__ = ["llama3_configs", "model_registry", "build_llama_config"]


def build_llama_config(*, dim: int, n_layers: int, n_heads: int, n_kv_heads: int | None, vocab_size: int,
                       multiple_of: int, ffn_dim_multiplier: float | None = None, rope_theta: float = 500000.0,
                       rope_scaling: str = "llama", max_context_length: int = 131072, weight_tying: bool = False,
                       norm_eps: float = 1e-5, depth_init: bool = True) -> Decoder.Config:
    hidden = ffn_hidden_dim(dim, multiple_of, ffn_dim_multiplier)
    head_dim = dim // n_heads
    layers = []
    for i in range(n_layers):
        out_std = 0.02 / math.sqrt(2 * (i + 1)) if depth_init else 0.02 / math.sqrt(2 * n_layers)
        layers.append(
            TransformerBlock.Config(
                layer_id=i,
                attention=GQAttention.Config(
                    dim=dim, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
                    wqkv=Linear.Config(init_std=0.02),
                    wo=Linear.Config(init_std=out_std),
                    rope=RoPE.Config(dim=head_dim, theta=rope_theta, style="complex", scaling=rope_scaling,
                                     max_context_length=max_context_length),
                ),
                feed_forward=FeedForward.Config(dim=dim, hidden_dim=hidden, w13=Linear.Config(init_std=0.02),
                                                w2=Linear.Config(init_std=out_std)),
                attention_norm=RMSNorm.Config(dim=dim, eps=norm_eps),
                ffn_norm=RMSNorm.Config(dim=dim, eps=norm_eps),
            )
        )
    return Decoder.Config(
        dim=dim, vocab_size=vocab_size, n_layers=n_layers, layers=layers,
        tok_embeddings=Embedding.Config(init_std=1.0),
        norm=RMSNorm.Config(dim=dim, eps=norm_eps),
        lm_head=Linear.Config(init_std=dim ** -0.5, init_cutoff=3.0),
        enable_weight_tying=weight_tying, max_context_length=max_context_length,
    )


llama3_configs = {
    "debugmodel": lambda: build_llama_config(dim=256, n_layers=6, n_heads=16, n_kv_heads=None, vocab_size=2048,
                                             multiple_of=256),
    # head dimension 128 with grouped queries: the shape the tcgen05 attention kernels are built for
    "debugmodel_hd128": lambda: build_llama_config(dim=512, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=2048,
                                                   multiple_of=256),
    "debugmodel_gqa": lambda: build_llama_config(dim=256, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=2048,
                                                 multiple_of=256),
    "1B": lambda: build_llama_config(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, vocab_size=128256,
                                     multiple_of=1024, ffn_dim_multiplier=1.5, weight_tying=True),
    "3B": lambda: build_llama_config(dim=3072, n_layers=28, n_heads=24, n_kv_heads=8, vocab_size=128256,
                                     multiple_of=1024, ffn_dim_multiplier=1.0, weight_tying=True),
    "8B": lambda: build_llama_config(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256,
                                     multiple_of=1024, ffn_dim_multiplier=1.3),
    "70B": lambda: build_llama_config(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, vocab_size=128256,
                                      multiple_of=4096, ffn_dim_multiplier=1.3),
    "405B": lambda: build_llama_config(dim=16384, n_layers=126, n_heads=128, n_kv_heads=8, vocab_size=128256,
                                       multiple_of=4096, ffn_dim_multiplier=1.2),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in llama3_configs:
        raise ValueError(f"unknown llama3 flavor '{flavor}' (have {sorted(llama3_configs)})")
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.parallel.pipeline import pipeline_decoder

    from .state_dict_adapter import Llama3StateDictAdapter

    return ModelSpec(name="llama3", flavor=flavor, model=llama3_configs[flavor](),
                     parallelize_fn=parallelize_decoder, pipelining_fn=pipeline_decoder,
                     state_dict_adapter=Llama3StateDictAdapter)
