"""Qwen3.5 checkpoint names and layouts (text decoder; parity: torchtitan/models/qwen3_5/state_dict_adapter.py).

Hugging Face files differ from the native layout in four places:

* Gated DeltaNet: one fused ``in_proj_qkv`` and one depthwise ``conv1d`` over ``[q | k | v]``; natively three
  projections and three convolution weights (``[C, 1, W]`` becomes ``[C, W]``);
* full attention: ``q_proj`` holds, per head, the query rows followed by the rows of the sigmoid output gate; natively
  the gate is its own projection (``o_gate``);
* MoE experts: fused ``gate_up_proj [E, 2F, D]`` and ``down_proj [E, D, F]`` tensors (or one 2-D tensor per expert in
  older exports); natively ``w1 / w3 [E, F, D]`` and ``w2 [E, D, F]``; the shared expert has a sigmoid gate;
* released multimodal checkpoints prefix the decoder with ``model.language_model.``, text-only exports with ``model.``:
  both are read, ``to_hf`` writes the prefix given by ``hf_prefix``;
* the vision tower (``model.visual.*``, read when the native model has one): the patch embedding is a 3-D
  convolution whose kernel equals the patch, natively a linear layer on the flattened patch; blocks are called
  ``blocks`` / ``attn.qkv`` / ``mlp.linear_fc1`` there and ``layers`` / ``wqkv`` / ``fc1`` here.
"""

from __future__ import annotations

import re

import torch

from torchtitan_b200.models.state_dict_adapter import StateDictAdapter

__all__ = ["Qwen35StateDictAdapter"]


_VISUAL = {
    "patch_embed.proj.bias": "patch_embed.bias",
    "pos_embed.weight": "pos_embed",
    "merger.norm.weight": "norm.weight", "merger.norm.bias": "norm.bias",
    "merger.linear_fc1.weight": "merger_fc1.weight", "merger.linear_fc1.bias": "merger_fc1.bias",
    "merger.linear_fc2.weight": "merger_fc2.weight", "merger.linear_fc2.bias": "merger_fc2.bias",
}
_VISUAL_BLOCK = {
    "norm1.weight": "norm1.weight", "norm1.bias": "norm1.bias", "norm2.weight": "norm2.weight", "norm2.bias": "norm2.bias",
    "attn.qkv.weight": "wqkv.weight", "attn.qkv.bias": "wqkv.bias", "attn.proj.weight": "proj.weight",
    "attn.proj.bias": "proj.bias", "mlp.linear_fc1.weight": "fc1.weight", "mlp.linear_fc1.bias": "fc1.bias",
    "mlp.linear_fc2.weight": "fc2.weight", "mlp.linear_fc2.bias": "fc2.bias",
}


class Qwen35StateDictAdapter(StateDictAdapter):
    hf_prefix = "model.language_model."

    hf_to_native = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.qkv_linear.wk.weight",
        "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.qkv_linear.wv.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.self_attn.q_norm.weight": "layers.{}.attention.q_norm.weight",
        "model.layers.{}.self_attn.k_norm.weight": "layers.{}.attention.k_norm.weight",
        "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
        "model.layers.{}.linear_attn.in_proj_z.weight": "layers.{}.attention.in_proj_z.weight",
        "model.layers.{}.linear_attn.in_proj_a.weight": "layers.{}.attention.in_proj_a.weight",
        "model.layers.{}.linear_attn.in_proj_b.weight": "layers.{}.attention.in_proj_b.weight",
        "model.layers.{}.linear_attn.A_log": "layers.{}.attention.A_log",
        "model.layers.{}.linear_attn.dt_bias": "layers.{}.attention.dt_bias",
        "model.layers.{}.linear_attn.norm.weight": "layers.{}.attention.norm_weight",
        "model.layers.{}.linear_attn.out_proj.weight": "layers.{}.attention.out_proj.weight",
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.mlp.gate.weight": "layers.{}.moe.router.gate.weight",
        "model.layers.{}.mlp.shared_expert.gate_proj.weight": "layers.{}.moe.shared_experts.w1.weight",
        "model.layers.{}.mlp.shared_expert.up_proj.weight": "layers.{}.moe.shared_experts.w3.weight",
        "model.layers.{}.mlp.shared_expert.down_proj.weight": "layers.{}.moe.shared_experts.w2.weight",
        "model.layers.{}.mlp.shared_expert_gate.weight": "layers.{}.moe.shared_gate.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "lm_head.weight",
    }

    # ------------------------------------------------------------------------------------------------------
    def _dims(self, layer: int):
        att = self.model_config.layers[layer].attention
        return att

    def from_hf(self, hf_state_dict):
        plain, out = {}, {}
        experts: dict[tuple[str, str], dict[int, torch.Tensor]] = {}
        for k, v in hf_state_dict.items():
            if k.startswith("model.language_model."):
                k = "model." + k[len("model.language_model."):]
            if k.startswith("model.visual."):
                if getattr(self.model_config, "vision_encoder", None) is None:
                    continue                               # a text-only native model: the tower is left out
                name = k[len("model.visual."):]
                mb = re.fullmatch(r"blocks\.(\d+)\.(.+)", name)
                if name == "patch_embed.proj.weight":
                    out["vision_encoder.patch_embed.weight"] = v.reshape(v.shape[0], -1)
                elif mb and mb.group(2) in _VISUAL_BLOCK:
                    out[f"vision_encoder.layers.{mb.group(1)}.{_VISUAL_BLOCK[mb.group(2)]}"] = v
                elif name in _VISUAL:
                    out["vision_encoder." + _VISUAL[name]] = v
                else:
                    raise KeyError(f"no native name for '{k}'")
                continue
            if k.startswith("mtp."):
                continue                                   # the multi-token-prediction head is not part of the decoder
            m = re.fullmatch(r"model\.layers\.(\d+)\.(.+)", k)
            rest = m.group(2) if m else None
            if rest == "linear_attn.in_proj_qkv.weight":
                i = int(m.group(1))
                a = self._dims(i)
                kd, vd = a.n_key_heads * a.key_head_dim, a.n_value_heads * a.value_head_dim
                q, kk, vv = v.split([kd, kd, vd], dim=0)
                out[f"layers.{i}.attention.in_proj_q.weight"] = q
                out[f"layers.{i}.attention.in_proj_k.weight"] = kk
                out[f"layers.{i}.attention.in_proj_v.weight"] = vv
            elif rest == "linear_attn.conv1d.weight":
                i = int(m.group(1))
                a = self._dims(i)
                kd, vd = a.n_key_heads * a.key_head_dim, a.n_value_heads * a.value_head_dim
                q, kk, vv = v.squeeze(1).split([kd, kd, vd], dim=0)
                out[f"layers.{i}.attention.conv_q"], out[f"layers.{i}.attention.conv_k"] = q, kk
                out[f"layers.{i}.attention.conv_v"] = vv
            elif rest == "self_attn.q_proj.weight":
                i = int(m.group(1))
                a = self._dims(i)
                w = v.view(a.n_heads, 2, a.head_dim, v.shape[-1])          # per head: query rows, then gate rows
                out[f"layers.{i}.attention.qkv_linear.wq.weight"] = w[:, 0].reshape(a.n_heads * a.head_dim, -1)
                out[f"layers.{i}.attention.o_gate.weight"] = w[:, 1].reshape(a.n_heads * a.head_dim, -1)
            elif rest == "mlp.experts.gate_up_proj":
                F_ = v.shape[1] // 2
                out[f"layers.{m.group(1)}.moe.routed_experts.inner_experts.w1_EFD"] = v[:, :F_]
                out[f"layers.{m.group(1)}.moe.routed_experts.inner_experts.w3_EFD"] = v[:, F_:]
            elif rest == "mlp.experts.down_proj":
                out[f"layers.{m.group(1)}.moe.routed_experts.inner_experts.w2_EDF"] = v
            elif rest is not None and re.fullmatch(r"mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight", rest):
                e, name = re.fullmatch(r"mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight", rest).groups()
                native = {"gate_proj": "w1_EFD", "up_proj": "w3_EFD", "down_proj": "w2_EDF"}[name]
                experts.setdefault((m.group(1), native), {})[int(e)] = v
            else:
                plain[k] = v
        out.update(super().from_hf(plain))
        for (layer, native), per in experts.items():
            out[f"layers.{layer}.moe.routed_experts.inner_experts.{native}"] = torch.stack([per[e] for e in range(len(per))])
        if self.model_config.enable_weight_tying and "lm_head.weight" not in out and "tok_embeddings.weight" in out:
            out["lm_head.weight"] = out["tok_embeddings.weight"]
        return out

    def to_hf(self, state_dict):
        plain, out = {}, {}
        visual: dict[str, torch.Tensor] = {}
        gdn: dict[str, dict[str, torch.Tensor]] = {}
        attn: dict[str, dict[str, torch.Tensor]] = {}
        moe: dict[str, dict[str, torch.Tensor]] = {}
        for k, v in state_dict.items():
            m = re.fullmatch(r"layers\.(\d+)\.attention\.(in_proj_[qkv]\.weight|conv_[qkv])", k)
            if m:
                gdn.setdefault(m.group(1), {})[m.group(2)] = v
                continue
            m = re.fullmatch(r"layers\.(\d+)\.attention\.(qkv_linear\.wq\.weight|o_gate\.weight)", k)
            if m:
                attn.setdefault(m.group(1), {})[m.group(2)] = v
                continue
            m = re.fullmatch(r"layers\.(\d+)\.moe\.routed_experts\.inner_experts\.(w1_EFD|w2_EDF|w3_EFD)", k)
            if m:
                moe.setdefault(m.group(1), {})[m.group(2)] = v
                continue
            if k.endswith("moe.expert_bias_E"):
                continue
            if k.startswith("vision_encoder."):
                name = k[len("vision_encoder."):]
                mb = re.fullmatch(r"layers\.(\d+)\.(.+)", name)
                inv_b = {b: a for a, b in _VISUAL_BLOCK.items()}
                inv = {b: a for a, b in _VISUAL.items()}
                if name == "patch_embed.weight":
                    vc = self.model_config.vision_encoder
                    visual[f"model.visual.patch_embed.proj.weight"] = v.reshape(
                        v.shape[0], vc.in_channels, vc.temporal_patch_size, vc.patch_size, vc.patch_size)
                elif mb and mb.group(2) in inv_b:
                    visual[f"model.visual.blocks.{mb.group(1)}.{inv_b[mb.group(2)]}"] = v
                elif name in inv:
                    visual["model.visual." + inv[name]] = v
                else:
                    raise KeyError(f"no Hugging Face name for '{k}'")
                continue
            plain[k] = v
        if self.model_config.enable_weight_tying:
            plain.pop("lm_head.weight", None)
        out.update(super().to_hf(plain))
        for i, d in gdn.items():
            out[f"model.layers.{i}.linear_attn.in_proj_qkv.weight"] = torch.cat(
                [d["in_proj_q.weight"], d["in_proj_k.weight"], d["in_proj_v.weight"]], dim=0)
            out[f"model.layers.{i}.linear_attn.conv1d.weight"] = torch.cat([d["conv_q"], d["conv_k"], d["conv_v"]], dim=0).unsqueeze(1)
        for i, d in attn.items():
            a = self._dims(int(i))
            q = d["qkv_linear.wq.weight"].view(a.n_heads, 1, a.head_dim, -1)
            g = d["o_gate.weight"].view(a.n_heads, 1, a.head_dim, -1)
            out[f"model.layers.{i}.self_attn.q_proj.weight"] = torch.cat([q, g], dim=1).reshape(2 * a.n_heads * a.head_dim, -1)
        for i, d in moe.items():
            out[f"model.layers.{i}.mlp.experts.gate_up_proj"] = torch.cat([d["w1_EFD"], d["w3_EFD"]], dim=1)
            out[f"model.layers.{i}.mlp.experts.down_proj"] = d["w2_EDF"]
        if self.hf_prefix != "model.":
            out = {(self.hf_prefix + k[len("model."):] if k.startswith("model.") else k): v for k, v in out.items()}
        out.update(visual)
        return out
