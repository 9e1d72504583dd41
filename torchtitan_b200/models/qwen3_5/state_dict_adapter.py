"""Qwen3.5 checkpoint names and layouts (text decoder; parity: torchtitan/models/qwen3_5/state_dict_adapter.py).

Hugging Face files differ from the native layout in four places:

* Gated DeltaNet: one fused ``in_proj_qkv`` and one depthwise ``conv1d`` over ``[q | k | v]``; natively three
  projections and three convolution weights (``[C, 1, W]`` becomes ``[C, W]``);
* full attention: ``q_proj`` holds, per head, the query rows followed by the rows of the sigmoid output gate; natively
  the gate is its own projection (``o_gate``);
* MoE experts: fused ``gate_up_proj [E, 2F, D]`` and ``down_proj [E, D, F]`` tensors (or one 2-D tensor per expert in
  older exports); natively ``w1 / w3 [E, F, D]`` and ``w2 [E, D, F]``; the shared expert has a sigmoid gate;
* released multimodal checkpoints prefix the decoder with ``model.language_model.``, text-only exports with ``model.``:
  both are read, ``to_hf`` writes the prefix given by ``hf_prefix``.
"""

from __future__ import annotations

import re

import torch

from torchtitan_b200.models.state_dict_adapter import StateDictAdapter

__all__ = ["Qwen35StateDictAdapter"]


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
            if k.startswith("model.visual.") or k.startswith("mtp."):
                continue                                   # the vision tower and the MTP head are not part of the decoder
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
        return out
