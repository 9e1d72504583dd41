"""Llama-3 checkpoint name mapping (parity: torchtitan/models/llama3/state_dict_adapter.py:19-154).

The native RoPE rotates adjacent pairs while Hugging Face rotates halves, so the
rows of ``wq``/``wk`` are re-ordered per head on the way in and out.
"""

from torchtitan_b200.models.state_dict_adapter import StateDictAdapter, halves_to_pairs, pairs_to_halves


class Llama3StateDictAdapter(StateDictAdapter):
    hf_to_native = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.qkv_linear.wq.weight",
        "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.qkv_linear.wk.weight",
        "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.qkv_linear.wv.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "lm_head.weight",
    }

    def _heads(self, key: str):
        attn = self.model_config.layers[0].attention
        if key.endswith("wq.weight"):
            return attn.n_heads
        if key.endswith("wk.weight"):
            return attn.n_kv_heads or attn.n_heads
        return None

    def transform_to_hf(self, native_key, tensor):
        h = self._heads(native_key)
        return pairs_to_halves(tensor, h) if h else tensor

    def transform_from_hf(self, native_key, tensor):
        h = self._heads(native_key)
        return halves_to_pairs(tensor, h) if h else tensor

    def to_hf(self, state_dict):
        sd = dict(state_dict)
        if self.model_config.enable_weight_tying:
            sd.pop("lm_head.weight", None)
        return super().to_hf(sd)

    def from_hf(self, hf_state_dict):
        out = super().from_hf(hf_state_dict)
        if self.model_config.enable_weight_tying and "lm_head.weight" not in out and "tok_embeddings.weight" in out:
            out["lm_head.weight"] = out["tok_embeddings.weight"]
        return out
