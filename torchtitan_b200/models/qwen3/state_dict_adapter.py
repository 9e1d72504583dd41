"""Qwen3 checkpoint names (parity: torchtitan/models/qwen3/state_dict_adapter.py).

Qwen's RoPE already uses the rotate-half convention, so no row permutation is needed.  MoE
experts are one 3-D tensor natively and one 2-D tensor per expert in Hugging Face files.
"""

import re

import torch

from torchtitan_b200.models.state_dict_adapter import StateDictAdapter

_EXPERT_KEYS = {
    "w1_EFD": "gate_proj", "w3_EFD": "up_proj", "w2_EDF": "down_proj",
}


class Qwen3StateDictAdapter(StateDictAdapter):
    hf_to_native = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.qkv_linear.wq.weight",
        "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.qkv_linear.wk.weight",
        "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.qkv_linear.wv.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.self_attn.q_norm.weight": "layers.{}.attention.q_norm.weight",
        "model.layers.{}.self_attn.k_norm.weight": "layers.{}.attention.k_norm.weight",
        "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.layers.{}.mlp.gate.weight": "layers.{}.moe.router.gate.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "lm_head.weight",
    }

    def to_hf(self, state_dict):
        plain, out = {}, {}
        for k, v in state_dict.items():
            m = re.fullmatch(r"layers\.(\d+)\.moe\.routed_experts\.inner_experts\.(w1_EFD|w2_EDF|w3_EFD)", k)
            if m:
                layer, name = m.group(1), _EXPERT_KEYS[m.group(2)]
                for e in range(v.shape[0]):
                    out[f"model.layers.{layer}.mlp.experts.{e}.{name}.weight"] = v[e]
            elif k.endswith("moe.expert_bias_E"):
                continue
            else:
                plain[k] = v
        if self.model_config.enable_weight_tying:
            plain.pop("lm_head.weight", None)
        out.update(super().to_hf(plain))
        return out

    def from_hf(self, hf_state_dict):
        plain, experts = {}, {}
        for k, v in hf_state_dict.items():
            m = re.fullmatch(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight", k)
            if m:
                native = {v2: k2 for k2, v2 in _EXPERT_KEYS.items()}[m.group(3)]
                experts.setdefault((m.group(1), native), {})[int(m.group(2))] = v
            else:
                plain[k] = v
        out = super().from_hf(plain)
        for (layer, native), per in experts.items():
            out[f"layers.{layer}.moe.routed_experts.inner_experts.{native}"] = torch.stack(
                [per[e] for e in range(len(per))])
        if self.model_config.enable_weight_tying and "lm_head.weight" not in out and "tok_embeddings.weight" in out:
            out["lm_head.weight"] = out["tok_embeddings.weight"]
        return out
