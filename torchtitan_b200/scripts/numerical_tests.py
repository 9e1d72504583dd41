"""Numerical parity between a Hugging Face ``transformers`` model and this framework's model on the same weights.

    python -m torchtitan_b200.scripts.numerical_tests --module llama3 --flavor 8B --hf-dir ./assets/hf/Llama-3.1-8B
    python -m torchtitan_b200.scripts.numerical_tests --module qwen3 --flavor debugmodel --random

The HF weights (a safetensors directory, or with ``--random`` a freshly initialised ``transformers`` model built from
the flavor's architecture) go through the family's state-dict adapter into the native model; both models then score
the same random token sequences and the script reports the mean KL divergence between their next-token
distributions and the largest logit difference.  Parity: scripts/checkpoint_conversion/numerical_tests_example.py
(same measure: KL divergence of the two logit sets).
"""

from __future__ import annotations

import argparse

import torch

from torchtitan_b200.models import get_model_spec

__all__ = ["hf_config_for", "hf_multimodal_config_for", "compare_multimodal", "checkpoint_state", "load_native_from_hf_state", "compare_logits", "compare_grads", "main"]


def hf_config_for(module: str, cfg):
    """A ``transformers`` config describing the same architecture as the native decoder config ``cfg``."""
    import transformers

    if module == "qwen3_5":
        full = next(b for b in cfg.layers if hasattr(b.attention, "rope"))
        lin = next(b for b in cfg.layers if not hasattr(b.attention, "rope"))
        fa, la = full.attention, lin.attention
        kw = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.dim, num_hidden_layers=len(cfg.layers),
                  num_attention_heads=fa.n_heads, num_key_value_heads=fa.n_kv_heads, head_dim=fa.head_dim,
                  linear_conv_kernel_dim=la.conv_kernel_size, linear_key_head_dim=la.key_head_dim,
                  linear_value_head_dim=la.value_head_dim, linear_num_key_heads=la.n_key_heads,
                  linear_num_value_heads=la.n_value_heads, rms_norm_eps=full.attention_norm.eps,
                  layer_types=["full_attention" if hasattr(b.attention, "rope") else "linear_attention" for b in cfg.layers],
                  rope_parameters=dict(rope_type="default", rope_theta=fa.rope.theta,
                                       partial_rotary_factor=fa.rope.dim / fa.head_dim),
                  max_position_embeddings=cfg.max_context_length, tie_word_embeddings=cfg.enable_weight_tying)
        if full.moe is not None:
            return transformers.Qwen3_5MoeTextConfig(
                moe_intermediate_size=full.moe.hidden_dim, shared_expert_intermediate_size=full.moe.shared_hidden_dim,
                num_experts=full.moe.num_experts, num_experts_per_tok=full.moe.top_k, **kw)
        return transformers.Qwen3_5TextConfig(intermediate_size=full.feed_forward.hidden_dim, **kw)
    blk = cfg.layers[0]
    att = blk.attention
    rope = att.rope
    common = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.dim, num_hidden_layers=len(cfg.layers),
                  num_attention_heads=att.n_heads, num_key_value_heads=getattr(att, "n_kv_heads", None) or att.n_heads,
                  rms_norm_eps=blk.attention_norm.eps, rope_theta=rope.theta, tie_word_embeddings=cfg.enable_weight_tying,
                  max_position_embeddings=min(cfg.max_context_length, 131072), attention_bias=False)
    inter = blk.feed_forward.hidden_dim if blk.feed_forward is not None else 0
    if module == "llama3":
        scaling = None
        if rope.scaling == "llama":
            scaling = dict(rope_type="llama3", factor=rope.scaling_factor, low_freq_factor=rope.low_freq_factor,
                           high_freq_factor=rope.high_freq_factor,
                           original_max_position_embeddings=getattr(rope, "original_max_context_length", 8192))
        return transformers.LlamaConfig(intermediate_size=inter, rope_scaling=scaling, head_dim=att.head_dim, **common)
    if module == "qwen3":
        if blk.moe is not None:
            return transformers.Qwen3MoeConfig(
                intermediate_size=blk.moe.hidden_dim, moe_intermediate_size=blk.moe.hidden_dim, head_dim=att.head_dim,
                num_experts=blk.moe.num_experts, num_experts_per_tok=blk.moe.top_k, norm_topk_prob=blk.moe.router.route_norm,
                decoder_sparse_step=1, mlp_only_layers=[], **common)
        return transformers.Qwen3Config(intermediate_size=inter, head_dim=att.head_dim, **common)
    if module == "gpt_oss":
        common.pop("attention_bias")
        yarn = dict(rope_type="yarn", factor=rope.rope_factor, original_max_position_embeddings=rope.original_seq_len,
                    beta_fast=rope.beta_fast, beta_slow=rope.beta_slow, truncate=False)
        window = next(b.attention.sliding_window for b in cfg.layers if b.attention.sliding_window)
        return transformers.GptOssConfig(
            intermediate_size=blk.moe.hidden_dim, head_dim=att.head_dim, num_local_experts=blk.moe.num_experts,
            num_experts_per_tok=blk.moe.top_k, sliding_window=window, rope_scaling=yarn, attention_bias=True,
            layer_types=["sliding_attention" if b.attention.sliding_window else "full_attention" for b in cfg.layers],
            **common)
    if module == "deepseek_v3":
        moe_blk = next(b for b in cfg.layers if b.moe is not None)
        moe, router = moe_blk.moe, moe_blk.moe.router
        if router.score_func != "sigmoid":
            raise ValueError("the Hugging Face DeepSeek-V3 model routes with sigmoid scores: use a flavor that does")
        n_dense = sum(1 for b in cfg.layers if b.moe is None)
        yarn = dict(rope_type="yarn", factor=rope.rope_factor, original_max_position_embeddings=rope.original_seq_len,
                    beta_fast=rope.beta_fast, beta_slow=rope.beta_slow, mscale=att.mscale, mscale_all_dim=att.mscale)
        return transformers.DeepseekV3Config(
            vocab_size=cfg.vocab_size, hidden_size=cfg.dim, num_hidden_layers=len(cfg.layers),
            intermediate_size=next(b for b in cfg.layers if b.moe is None).feed_forward.hidden_dim,
            moe_intermediate_size=moe.hidden_dim, num_attention_heads=att.n_heads, num_key_value_heads=att.n_heads,
            n_shared_experts=moe.shared_hidden_dim // moe.hidden_dim, n_routed_experts=moe.num_experts,
            routed_scaling_factor=router.route_scale, kv_lora_rank=att.kv_lora_rank, q_lora_rank=att.q_lora_rank or None,
            qk_rope_head_dim=att.qk_rope_head_dim, v_head_dim=att.v_head_dim, qk_nope_head_dim=att.qk_nope_head_dim,
            n_group=router.num_expert_groups or 1, topk_group=router.num_limited_groups or 1,
            num_experts_per_tok=moe.top_k, first_k_dense_replace=n_dense, norm_topk_prob=router.route_norm,
            rms_norm_eps=blk.attention_norm.eps, rope_theta=rope.theta, rope_scaling=yarn,
            max_position_embeddings=cfg.max_context_length, tie_word_embeddings=False, attention_bias=False)
    raise ValueError(f"no Hugging Face config mapping for module '{module}'")


def checkpoint_state(hf_model) -> dict[str, torch.Tensor]:
    """The tensors of ``hf_model`` under their checkpoint names (``save_pretrained`` undoes the in-memory fusion of
    expert weights that recent ``transformers`` releases apply on load)."""
    import os
    import tempfile

    from safetensors import safe_open

    out = {}
    with tempfile.TemporaryDirectory() as d:
        hf_model.save_pretrained(d, safe_serialization=True)
        for fn in sorted(f for f in os.listdir(d) if f.endswith(".safetensors")):
            with safe_open(os.path.join(d, fn), framework="pt", device="cpu") as f:
                for k in f.keys():
                    out[k] = f.get_tensor(k)
    if any(".language_model.language_model." in k for k in out):
        # composite (vision + text) models built from a config: the name conversion of ``save_pretrained`` repeats the
        # prefix; their in-memory names already are the released checkpoint names
        return {k: v.detach().clone() for k, v in hf_model.state_dict().items()}
    return out


def load_native_from_hf_state(spec, hf_state: dict[str, torch.Tensor], hf_dir: str | None = None):
    """The native model (fp32, CPU) with the weights of ``hf_state`` (Hugging Face names)."""
    from torchtitan_b200.models.common.module import iter_checkpoint_slices

    adapter = spec.state_dict_adapter(spec.model, hf_dir)
    native = adapter.from_hf(dict(hf_state))
    model = spec.model.build()
    fused = dict(iter_checkpoint_slices(model))
    with torch.no_grad():
        for k, p in model.named_parameters():
            if k in fused:
                for name, a, b in fused[k]:
                    p[a:b].copy_(native[name].float())
            else:
                p.copy_(native[k].float())
    model.init_buffers() if hasattr(model, "init_buffers") else None
    return model.float().eval()


@torch.no_grad()
def compare_logits(native, hf_model, tokens: torch.Tensor) -> dict:
    """``tokens [B, T]``: mean KL(hf || native) over positions and the largest absolute logit difference."""
    kls, worst = [], 0.0
    for row in tokens:
        ours = native(row, torch.arange(row.shape[0])).float()
        theirs = hf_model(input_ids=row[None]).logits[0].float()
        lp, lq = torch.log_softmax(theirs, -1), torch.log_softmax(ours, -1)
        kls.append(float((lp.exp() * (lp - lq)).sum(-1).mean()))
        worst = max(worst, float((ours - theirs).abs().max()))
    return {"kl_mean": sum(kls) / len(kls), "max_abs_logit_diff": worst}


def compare_grads(spec, native, hf_model, tokens: torch.Tensor) -> dict:
    """Gradients of the summed next-token cross entropy on ``tokens [B, T]``: the native gradients, renamed and
    re-laid-out by the state-dict adapter, against ``transformers`` autograd.  Compares the parameters whose Hugging
    Face checkpoint name is also an in-memory parameter name (fused expert tensors of recent releases are skipped)."""
    from torchtitan_b200.models.common.module import iter_checkpoint_slices

    for m in (native, hf_model):
        m.zero_grad(set_to_none=True)
        m.train(False)
    for row in tokens:
        inp, lab = row[:-1], row[1:]
        torch.nn.functional.cross_entropy(native(inp, torch.arange(inp.shape[0])).float(), lab, reduction="sum").backward()
        torch.nn.functional.cross_entropy(hf_model(input_ids=inp[None]).logits[0].float(), lab, reduction="sum").backward()
    fused = dict(iter_checkpoint_slices(native))
    grads = {}
    for k, p in native.named_parameters():
        if p.grad is None:
            continue
        if k in fused:
            for name, a, b in fused[k]:
                grads[name] = p.grad[a:b]
        else:
            grads[k] = p.grad
    adapter = spec.state_dict_adapter(spec.model, None)
    if hasattr(adapter, "hf_prefix"):
        adapter.hf_prefix = "model."
    as_hf = adapter.to_hf(grads)
    theirs = {k: p.grad for k, p in hf_model.named_parameters() if p.grad is not None}
    worst, n = 0.0, 0
    for k, g in as_hf.items():
        if k in theirs and theirs[k].shape == g.shape:
            denom = float(theirs[k].abs().max()) + 1e-12
            worst = max(worst, float((g - theirs[k]).abs().max()) / denom)
            n += 1
    return {"grad_tensors_compared": n, "max_rel_grad_diff": worst}


def hf_multimodal_config_for(module: str, cfg):
    """The ``transformers`` config of a vision-language flavor (Qwen3.5: ViT tower + interleaved three-axis RoPE)."""
    import transformers

    if module != "qwen3_5":
        raise ValueError(f"no Hugging Face multimodal mapping for module '{module}'")
    text = hf_config_for(module, cfg)
    full = next(b for b in cfg.layers if hasattr(b.attention, "rope"))
    text.rope_parameters["mrope_section"] = list(full.attention.rope.mrope_sections)
    text.rope_parameters["mrope_interleaved"] = True
    vis = cfg.vision_encoder
    vision = dict(depth=len(vis.layers) or vis.n_layers, hidden_size=vis.dim, intermediate_size=vis.mlp_dim,
                  num_heads=vis.num_heads, in_channels=vis.in_channels, patch_size=vis.patch_size,
                  spatial_merge_size=vis.spatial_merge, temporal_patch_size=vis.temporal_patch_size,
                  out_hidden_size=cfg.dim, num_position_embeddings=vis.num_position_embeddings)
    top = cfg.vocab_size
    return transformers.Qwen3_5Config(text_config=text.to_dict(), vision_config=vision, image_token_id=cfg.image_token_id,
                                      vision_start_token_id=top - 3, vision_end_token_id=top - 2, video_token_id=top - 4,
                                      tie_word_embeddings=cfg.enable_weight_tying)


@torch.no_grad()
def compare_multimodal(spec, native, hf_model, grids=((4, 6), (2, 4)), seed: int = 0) -> dict:
    """Logits on text interleaved with images of the given patch grids.  The native tower takes row-major single-frame
    patches; ``transformers`` takes two-frame patches in merge-window order (what its processor emits)."""
    cfg = spec.model
    vis = cfg.vision_encoder
    g = torch.Generator().manual_seed(seed)
    m, P2 = vis.spatial_merge, vis.patch_size ** 2
    start, end = cfg.vocab_size - 3, cfg.vocab_size - 2
    low = cfg.vocab_size - 8

    def window(x, h, w):
        return x.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)

    parts, rowmajor, windowed = [torch.randint(0, low, (10,), generator=g)], [], []
    for gh, gw in grids:
        parts += [torch.tensor([start]), torch.full((gh * gw // (m * m),), cfg.image_token_id), torch.tensor([end]),
                  torch.randint(0, low, (7,), generator=g)]
        p = torch.randn(gh * gw, vis.in_channels * P2, generator=g)
        rowmajor.append(p)
        frames = p.view(-1, vis.in_channels, 1, P2).expand(-1, -1, vis.temporal_patch_size, -1).reshape(gh * gw, -1)
        windowed.append(window(frames, gh, gw))
    tok = torch.cat(parts)
    theirs = hf_model(input_ids=tok[None], pixel_values=torch.cat(windowed),
                      image_grid_thw=torch.tensor([[1, h, w] for h, w in grids]),
                      mm_token_type_ids=(tok == cfg.image_token_id).long()[None]).logits[0].float()
    ours = native(tok, torch.arange(tok.shape[0]), pixel_patches=torch.cat(rowmajor), grid_hw=torch.tensor(grids)).float()
    lp, lq = torch.log_softmax(theirs, -1), torch.log_softmax(ours, -1)
    return {"kl_mean": float((lp.exp() * (lp - lq)).sum(-1).mean()), "max_abs_logit_diff": float((ours - theirs).abs().max())}


def main(argv=None) -> dict:
    import transformers

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--module", required=True)
    ap.add_argument("--flavor", required=True)
    ap.add_argument("--hf-dir", default=None)
    ap.add_argument("--random", action="store_true", help="compare on a freshly initialised transformers model")
    ap.add_argument("--perturb", type=float, default=0.0,
                    help="with --random: noise added to every 1-D parameter (norm gains, biases, sinks, decay terms), "
                         "which a fresh initialisation leaves at 0 or 1")
    ap.add_argument("--grads", action="store_true", help="also compare the gradients of a cross-entropy loss")
    ap.add_argument("--seq-len", type=int, default=64)
    ap.add_argument("--num-seqs", type=int, default=4)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    if bool(args.hf_dir) == bool(args.random):
        raise SystemExit("give exactly one of --hf-dir and --random")
    spec = get_model_spec(args.module, args.flavor)
    torch.manual_seed(args.seed)
    multimodal = getattr(spec.model, "vision_encoder", None) is not None
    if args.random and multimodal:
        hf_model = transformers.AutoModelForImageTextToText.from_config(
            hf_multimodal_config_for(args.module, spec.model)).float().eval()
    elif args.random:
        hf_model = transformers.AutoModelForCausalLM.from_config(hf_config_for(args.module, spec.model)).float().eval()
    if args.random:
        if args.perturb:
            with torch.no_grad():
                for p in hf_model.parameters():
                    if p.dim() == 1:
                        p.add_(torch.randn_like(p) * args.perturb)
    elif multimodal:
        hf_model = transformers.AutoModelForImageTextToText.from_pretrained(args.hf_dir, torch_dtype=torch.float32).eval()
    else:
        hf_model = transformers.AutoModelForCausalLM.from_pretrained(args.hf_dir, torch_dtype=torch.float32).eval()
    native = load_native_from_hf_state(spec, checkpoint_state(hf_model), args.hf_dir)
    if multimodal:
        res = compare_multimodal(spec, native, hf_model, seed=args.seed)
        print(f"{args.module} {args.flavor} (text + images): mean KL {res['kl_mean']:.3e}, largest logit difference "
              f"{res['max_abs_logit_diff']:.3e}")
        return res
    g = torch.Generator().manual_seed(args.seed)
    tokens = torch.randint(0, spec.model.vocab_size, (args.num_seqs, args.seq_len), generator=g)
    res = compare_logits(native, hf_model, tokens)
    print(f"{args.module} {args.flavor}: mean KL {res['kl_mean']:.3e}, largest logit difference {res['max_abs_logit_diff']:.3e}")
    if args.grads:
        res.update(compare_grads(spec, native, hf_model, tokens))
        print(f"gradients: {res['grad_tensors_compared']} tensors, largest relative difference {res['max_rel_grad_diff']:.3e}")
    return res


if __name__ == "__main__":
    main()
