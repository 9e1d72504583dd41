"""Kimi / Moonlight family: DeepSeek-V3 style decoders (multi-head latent attention, shared
experts, sigmoid routing) with Moonshot's hyper-parameters.  Flavors: debugmodel, moonlight
(16B-A3B) and kimi_k2 (1T-A32B); parity: torchtitan/models/kimi_k2_7/__init__.py.  The training
recipes put the matrix parameters on DistMuon (``config_registry.kimi_muon_optimizer``) and the rest
on AdamW.  The vision tower of the VL flavors is not built here.
"""

from __future__ import annotations

from torchtitan_b200.models.deepseek_v3 import build_deepseek_v3_config
from torchtitan_b200.models.spec import ModelSpec

__all__ = ["kimi_configs", "model_registry"]

kimi_configs = {
    "debugmodel": lambda: build_deepseek_v3_config(
        vocab_size=2048, dim=256, inter_dim=1024, moe_inter_dim=256, n_layers=4, n_dense_layers=1, n_heads=8,
        n_routed_experts=8, n_shared_experts=1, n_activated_experts=2, score_func="sigmoid", route_norm=True,
        route_scale=2.446, rope_theta=50000.0, rope_factor=1.0, mscale=1.0),
    "moonlight": lambda: build_deepseek_v3_config(
        vocab_size=163840, dim=2048, inter_dim=11264, moe_inter_dim=1408, n_layers=27, n_dense_layers=1, n_heads=16,
        n_routed_experts=64, n_shared_experts=2, n_activated_experts=6, score_func="sigmoid", route_norm=True,
        route_scale=2.446, rope_theta=50000.0, rope_factor=1.0, mscale=1.0, max_context_length=8192),
    "kimi_k2": lambda: build_deepseek_v3_config(
        vocab_size=163840, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=61, n_dense_layers=1, n_heads=64,
        n_routed_experts=384, n_shared_experts=1, n_activated_experts=8, score_func="sigmoid", route_norm=True,
        route_scale=2.827, q_lora_rank=1536, rope_theta=50000.0, rope_factor=32.0, mscale=1.0, max_context_length=4096),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in kimi_configs:
        raise ValueError(f"unknown kimi_k2_7 flavor '{flavor}' (have {sorted(kimi_configs)})")
    from torchtitan_b200.models.deepseek_v3.state_dict_adapter import DeepSeekV3StateDictAdapter
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.parallel.pipeline import pipeline_decoder

    return ModelSpec(name="kimi_k2_7", flavor=flavor, model=kimi_configs[flavor](), parallelize_fn=parallelize_decoder,
                     pipelining_fn=pipeline_decoder, state_dict_adapter=DeepSeekV3StateDictAdapter)
