"""GPT-OSS checkpoint names (parity: torchtitan/models/gpt_oss/state_dict_adapter.py)."""

from torchtitan_b200.models.state_dict_adapter import StateDictAdapter


class GptOssStateDictAdapter(StateDictAdapter):
    hf_to_native = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.qkv_linear.wq.weight",
        "model.layers.{}.self_attn.q_proj.bias": "layers.{}.attention.qkv_linear.wq.bias",
        "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.qkv_linear.wk.weight",
        "model.layers.{}.self_attn.k_proj.bias": "layers.{}.attention.qkv_linear.wk.bias",
        "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.qkv_linear.wv.weight",
        "model.layers.{}.self_attn.v_proj.bias": "layers.{}.attention.qkv_linear.wv.bias",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.self_attn.o_proj.bias": "layers.{}.attention.wo.bias",
        "model.layers.{}.self_attn.sinks": "layers.{}.attention.sinks",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.layers.{}.mlp.router.weight": "layers.{}.moe.router.gate.weight",
        "model.layers.{}.mlp.router.bias": "layers.{}.moe.router.gate.bias",
        "model.layers.{}.mlp.experts.gate_up_proj": "layers.{}.moe.routed_experts.inner_experts.mlp1_weight",
        "model.layers.{}.mlp.experts.gate_up_proj_bias": "layers.{}.moe.routed_experts.inner_experts.mlp1_bias",
        "model.layers.{}.mlp.experts.down_proj": "layers.{}.moe.routed_experts.inner_experts.mlp2_weight",
        "model.layers.{}.mlp.experts.down_proj_bias": "layers.{}.moe.routed_experts.inner_experts.mlp2_bias",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "lm_head.weight",
    }

    # Hugging Face stores the expert matrices as [E, in, out]; natively they are [E, out, in].
    def transform_to_hf(self, native_key, tensor):
        if native_key.endswith("mlp1_weight") or native_key.endswith("mlp2_weight"):
            return tensor.transpose(-2, -1).contiguous()
        return tensor

    def transform_from_hf(self, native_key, tensor):
        if native_key.endswith("mlp1_weight") or native_key.endswith("mlp2_weight"):
            return tensor.transpose(-2, -1).contiguous()
        return tensor

    def to_hf(self, state_dict):
        return super().to_hf({k: v for k, v in state_dict.items() if not k.endswith("moe.expert_bias_E")})
