"""Kimi / Moonlight family: DeepSeek-V3 style decoders (multi-head latent attention, shared
experts, sigmoid routing) with Moonshot's hyper-parameters.  Flavors: debugmodel, moonlight
(16B-A3B) and kimi_k2 (1T-A32B); parity: torchtitan/models/kimi_k2_7/__init__.py.  The training
recipes put the matrix parameters on DistMuon (``config_registry.kimi_muon_optimizer``) and the rest
on AdamW.  The VL flavors (``debugmodel_vl``, ``kimi_vl_a3b``) put the shared ViT tower
(``models/common/vision_encoder.py``) in front of the text decoder.
"""

from __future__ import annotations

from torchtitan_b200.models.deepseek_v3 import build_deepseek_v3_config
from torchtitan_b200.models.spec import ModelSpec

__all__ = ["kimi_configs", "model_registry"]

def _vl(text_cfg, *, dim, heads, mlp, layers, patch, image_token_id):
    from torchtitan_b200.models.common.multimodal import to_multimodal
    from torchtitan_b200.models.common.vision_encoder import VisionEncoder

    vis = VisionEncoder.Config(patch_size=patch, dim=dim, num_heads=heads, mlp_dim=mlp, n_layers=layers, spatial_merge=2)
    return to_multimodal(text_cfg, vis, image_token_id)


kimi_configs = {
    "debugmodel": lambda: build_deepseek_v3_config(
        vocab_size=2048, dim=256, inter_dim=1024, moe_inter_dim=256, n_layers=4, n_dense_layers=1, n_heads=8,
        n_routed_experts=8, n_shared_experts=1, n_activated_experts=2, score_func="sigmoid", route_norm=True,
        route_scale=2.446, rope_theta=50000.0, rope_factor=1.0, mscale=1.0),
    "debugmodel_vl": lambda: _vl(kimi_configs["debugmodel"](), dim=64, heads=2, mlp=128, layers=2, patch=4,
                                 image_token_id=2047),
    "kimi_vl_a3b": lambda: _vl(kimi_configs["moonlight"](), dim=1152, heads=16, mlp=4304, layers=27, patch=14,
                               image_token_id=163605),
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
