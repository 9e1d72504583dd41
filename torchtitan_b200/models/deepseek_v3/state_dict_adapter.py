"""DeepSeek-V3 checkpoint names (parity: torchtitan/models/deepseek_v3/state_dict_adapter.py).
Routed experts are one 3-D tensor natively and one 2-D tensor per expert in Hugging Face files."""

from torchtitan_b200.models.qwen3.state_dict_adapter import Qwen3StateDictAdapter


class DeepSeekV3StateDictAdapter(Qwen3StateDictAdapter):
    hf_to_native = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
        "model.layers.{}.self_attn.q_a_proj.weight": "layers.{}.attention.wq_a.weight",
        "model.layers.{}.self_attn.q_a_layernorm.weight": "layers.{}.attention.q_norm.weight",
        "model.layers.{}.self_attn.q_b_proj.weight": "layers.{}.attention.wq_b.weight",
        "model.layers.{}.self_attn.kv_a_proj_with_mqa.weight": "layers.{}.attention.wkv_a.weight",
        "model.layers.{}.self_attn.kv_a_layernorm.weight": "layers.{}.attention.kv_norm.weight",
        "model.layers.{}.self_attn.kv_b_proj.weight": "layers.{}.attention.wkv_b.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.mlp.shared_experts.gate_proj.weight": "layers.{}.moe.shared_experts.w1.weight",
        "model.layers.{}.mlp.shared_experts.up_proj.weight": "layers.{}.moe.shared_experts.w3.weight",
        "model.layers.{}.mlp.shared_experts.down_proj.weight": "layers.{}.moe.shared_experts.w2.weight",
        "model.layers.{}.mlp.gate.weight": "layers.{}.moe.router.gate.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "lm_head.weight",
    }

    def to_hf(self, state_dict):
        bias = {k: v for k, v in state_dict.items() if k.endswith("moe.expert_bias_E")}
        out = super().to_hf(state_dict)
        for k, v in bias.items():
            layer = k.split(".")[1]
            out[f"model.layers.{layer}.mlp.gate.e_score_correction_bias"] = v
        return out

    def from_hf(self, hf_state_dict):
        rest, bias = {}, {}
        for k, v in hf_state_dict.items():
            if k.endswith("mlp.gate.e_score_correction_bias"):
                bias[f"layers.{k.split('.')[2]}.moe.expert_bias_E"] = v
            else:
                rest[k] = v
        out = super().from_hf(rest)
        out.update(bias)
        return out
