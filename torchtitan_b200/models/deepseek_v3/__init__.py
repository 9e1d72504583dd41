"""DeepSeek-V3 family: multi-head latent attention, dense first layers, then MoE layers with
shared experts and (for the large models) group-limited sigmoid routing.

Hyper-parameters follow torchtitan/models/deepseek_v3/__init__.py (flavors debugmodel, 16B,
236B, 671B); the decoder and MoE blocks are the shared ones of ``models.common``.
"""

from __future__ import annotations

from torchtitan_b200.models.common.decoder import Decoder, TransformerBlock
from torchtitan_b200.models.common.layers import Embedding, FeedForward, Linear, RMSNorm, RoPE
from torchtitan_b200.models.common.mla import MLAttention
from torchtitan_b200.models.common.moe import GroupedExperts, MoE, RoutedExperts, TokenChoiceTopKRouter
from torchtitan_b200.models.spec import ModelSpec

__all__ = ["deepseek_v3_configs", "model_registry", "build_deepseek_v3_config"]

_EPS = 1e-6


def build_deepseek_v3_config(*, vocab_size, dim, inter_dim, moe_inter_dim, n_layers, n_dense_layers, n_heads,
                             n_routed_experts, n_shared_experts, n_activated_experts, n_expert_groups=1,
                             n_limited_groups=1, score_func="softmax", route_scale=1.0, route_norm=False,
                             q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                             mscale=0.70, rope_theta=10000.0, rope_factor=40.0, original_seq_len=4096,
                             max_context_length=4096, load_balance_coeff=1e-3, n_mtp_layers=0, mtp_scale=0.3) -> Decoder.Config:
    layers = []
    for i in range(n_layers + n_mtp_layers):
        out_std = 0.02 / (2 * (i + 1)) ** 0.5
        attn = MLAttention.Config(
            dim=dim, n_heads=n_heads, q_lora_rank=q_lora_rank, kv_lora_rank=kv_lora_rank,
            qk_nope_head_dim=qk_nope_head_dim, qk_rope_head_dim=qk_rope_head_dim, v_head_dim=v_head_dim,
            norm_eps=_EPS, mscale=mscale, out_init_std=out_std,
            rope=RoPE.Config(dim=qk_rope_head_dim, theta=rope_theta, style="complex", scaling="yarn",
                             rope_factor=rope_factor, original_seq_len=original_seq_len,
                             max_context_length=max_context_length))
        ff = moe = None
        if i < n_dense_layers:
            ff = FeedForward.Config(dim=dim, hidden_dim=inter_dim, w13=Linear.Config(init_std=0.02),
                                    w2=Linear.Config(init_std=out_std))
        else:
            moe = MoE.Config(
                dim=dim, hidden_dim=moe_inter_dim, num_experts=n_routed_experts, top_k=n_activated_experts,
                router=TokenChoiceTopKRouter.Config(
                    score_func=score_func, route_norm=route_norm, route_scale=route_scale,
                    num_expert_groups=n_expert_groups if n_expert_groups > 1 else None,
                    num_limited_groups=n_limited_groups if n_expert_groups > 1 else None),
                routed_experts=RoutedExperts.Config(inner_experts=GroupedExperts.Config(init_std=0.02, out_init_std=out_std)),
                shared_hidden_dim=n_shared_experts * moe_inter_dim,
                shared_experts=FeedForward.Config(w13=Linear.Config(init_std=0.02), w2=Linear.Config(init_std=out_std)),
                load_balance_coeff=load_balance_coeff)
        common = dict(layer_id=i, attention=attn, feed_forward=ff, moe=moe,
                      attention_norm=RMSNorm.Config(dim=dim, eps=_EPS), ffn_norm=RMSNorm.Config(dim=dim, eps=_EPS))
        if i < n_layers:
            layers.append(TransformerBlock.Config(**common))
        else:   # multi-token prediction depths: a regular block behind the embedding / hidden fusion
            from .mtp import MTPBlock

            layers.append(MTPBlock.Config(**common, dim=dim, enorm=RMSNorm.Config(dim=dim, eps=_EPS),
                                          hnorm=RMSNorm.Config(dim=dim, eps=_EPS), mtp_norm=RMSNorm.Config(dim=dim, eps=_EPS),
                                          eh_proj=Linear.Config(init_std=0.02)))
    base = dict(dim=dim, vocab_size=vocab_size, n_layers=n_layers, layers=layers[:n_layers],
                tok_embeddings=Embedding.Config(init_std=1.0), norm=RMSNorm.Config(dim=dim, eps=_EPS),
                lm_head=Linear.Config(init_std=dim ** -0.5, init_cutoff=3.0), max_context_length=max_context_length)
    if n_mtp_layers:
        from .mtp import MTPDecoder

        return MTPDecoder.Config(**base, mtp_layers=layers[n_layers:], mtp_scale=mtp_scale)
    return Decoder.Config(**base)


deepseek_v3_configs = {
    "debugmodel": lambda: build_deepseek_v3_config(
        vocab_size=2048, dim=256, inter_dim=1024, moe_inter_dim=256, n_layers=6, n_dense_layers=1, n_heads=16,
        n_routed_experts=8, n_shared_experts=2, n_activated_experts=3, route_scale=1.0),
    # the routing of the released V3 models at toy size: sigmoid scores, normalised top-k inside two of four groups
    "debugmodel_v3routing": lambda: build_deepseek_v3_config(
        vocab_size=2048, dim=128, inter_dim=256, moe_inter_dim=64, n_layers=3, n_dense_layers=1, n_heads=4,
        n_routed_experts=8, n_shared_experts=1, n_activated_experts=2, n_expert_groups=4, n_limited_groups=2,
        score_func="sigmoid", route_norm=True, route_scale=2.5, kv_lora_rank=64, qk_nope_head_dim=32,
        qk_rope_head_dim=16, v_head_dim=32, q_lora_rank=48, max_context_length=8192),
    "debugmodel_mtp": lambda: build_deepseek_v3_config(
        vocab_size=2048, dim=256, inter_dim=1024, moe_inter_dim=256, n_layers=3, n_dense_layers=1, n_heads=16,
        n_routed_experts=8, n_shared_experts=2, n_activated_experts=3, route_scale=1.0, n_mtp_layers=2),
    "16B": lambda: build_deepseek_v3_config(
        vocab_size=102400, dim=2048, inter_dim=10944, moe_inter_dim=1408, n_layers=27, n_dense_layers=1, n_heads=16,
        n_routed_experts=64, n_shared_experts=2, n_activated_experts=6, route_scale=1.0),
    "236B": lambda: build_deepseek_v3_config(
        vocab_size=102400, dim=5120, inter_dim=12288, moe_inter_dim=1536, n_layers=60, n_dense_layers=1, n_heads=128,
        n_routed_experts=160, n_shared_experts=2, n_activated_experts=6, n_expert_groups=8, n_limited_groups=3,
        route_scale=16.0, q_lora_rank=1536),
    "671B": lambda: build_deepseek_v3_config(
        vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=61, n_dense_layers=3, n_heads=128,
        n_routed_experts=256, n_shared_experts=1, n_activated_experts=8, n_expert_groups=8, n_limited_groups=4,
        score_func="sigmoid", route_norm=True, route_scale=2.5, q_lora_rank=1536, mscale=1.0),
    "671B_mtp": lambda: build_deepseek_v3_config(
        vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=61, n_dense_layers=3, n_heads=128,
        n_routed_experts=256, n_shared_experts=1, n_activated_experts=8, n_expert_groups=8, n_limited_groups=4,
        score_func="sigmoid", route_norm=True, route_scale=2.5, q_lora_rank=1536, mscale=1.0, n_mtp_layers=1),
}


def model_registry(flavor: str) -> ModelSpec:
    if flavor not in deepseek_v3_configs:
        raise ValueError(f"unknown deepseek_v3 flavor '{flavor}' (have {sorted(deepseek_v3_configs)})")
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.parallel.pipeline import pipeline_decoder

    from .state_dict_adapter import DeepSeekV3StateDictAdapter

    return ModelSpec(name="deepseek_v3", flavor=flavor, model=deepseek_v3_configs[flavor](),
                     parallelize_fn=parallelize_decoder, pipelining_fn=pipeline_decoder,
                     state_dict_adapter=DeepSeekV3StateDictAdapter)
