"""Train a Hugging Face causal-LM architecture with this framework's engine, parallelisms and data pipeline::

    python -m torchtitan_b200.experiments.transformers_backend.train --hf-model debug_llama --steps 20
    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 -m torchtitan_b200.experiments.transformers_backend.train \\
        --hf-model ./assets/hf/Qwen3-30B-A3B --native-moe --parallelism.tensor_parallel_degree 2 --steps 100

``--hf-model`` is a registered debug architecture (``debug_llama``, ``debug_qwen3_moe``, ``debug_deepseek_v3``) or a
folder with a ``config.json`` (random init; add ``--load-weights`` to read its safetensors).  Everything after the
backend's own flags is parsed like the regular trainer's command line (``--parallelism.*``, ``--training.*``,
``--optimizer.lr``, ``--dataloader.dataset`` ...).  Data-parallel sharding and tensor parallelism go through
``parallelize_hf``, pipeline parallelism through ``pipeline_hf``; ``--native-moe`` swaps the expert blocks for the
native MoE layer first.

Parity: torchtitan/experiments/transformers_modeling_backend/{trainer.py:15-76, config_registry.py:29-286,
__init__.py:22-172} (there a model spec plugged into the regular trainer).
"""

from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist

from torchtitan_b200.utils.logging import init_logger, logger

from . import HFCausalLM, hf_pipeline_train_steps, parallelize_hf, pipeline_hf

__all__ = ["DEBUG_MODELS", "hf_config", "main"]


def _debug_llama():
    import transformers

    return transformers.LlamaConfig(vocab_size=2048, hidden_size=256, intermediate_size=768, num_hidden_layers=6,
                                    num_attention_heads=16, num_key_value_heads=8, max_position_embeddings=2048,
                                    tie_word_embeddings=False)


def _debug_qwen3_moe():
    import transformers

    return transformers.Qwen3MoeConfig(vocab_size=2048, hidden_size=256, intermediate_size=768, moe_intermediate_size=128,
                                       num_hidden_layers=4, num_attention_heads=16, num_key_value_heads=8, head_dim=16,
                                       num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                                       mlp_only_layers=[], max_position_embeddings=2048)


def _debug_deepseek_v3():
    import transformers

    return transformers.DeepseekV3Config(vocab_size=2048, hidden_size=256, intermediate_size=768, moe_intermediate_size=128,
                                         num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=8, n_routed_experts=8,
                                         n_shared_experts=1, num_experts_per_tok=3, n_group=4, topk_group=2,
                                         routed_scaling_factor=2.5, norm_topk_prob=True, first_k_dense_replace=1,
                                         q_lora_rank=64, kv_lora_rank=64, qk_nope_head_dim=16, qk_rope_head_dim=16,
                                         v_head_dim=16, max_position_embeddings=2048)


DEBUG_MODELS = {"debug_llama": _debug_llama, "debug_qwen3_moe": _debug_qwen3_moe, "debug_deepseek_v3": _debug_deepseek_v3}


def hf_config(name_or_path: str):
    if name_or_path in DEBUG_MODELS:
        return DEBUG_MODELS[name_or_path]()
    from transformers import AutoConfig

    if not os.path.isdir(name_or_path):
        raise ValueError(f"--hf-model: '{name_or_path}' is neither a folder nor one of {sorted(DEBUG_MODELS)}")
    return AutoConfig.from_pretrained(name_or_path)


def _synthetic(vocab: int, tokens: int, ctx: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    while True:
        ids = torch.randint(0, vocab, (tokens + 1,), generator=g)
        pos = torch.arange(tokens) % ctx
        yield ids[:-1], pos, ids[1:]


def main(argv: list[str] | None = None) -> list[float]:
    from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.parallel import utils as dist_utils
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.utils.device import get_local_device

    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--hf-model", default="debug_llama")
    ap.add_argument("--native-moe", action="store_true")
    ap.add_argument("--load-weights", action="store_true")
    ap.add_argument("--steps", type=int, default=10)
    own, rest = ap.parse_known_args(argv)
    job = ConfigManager().parse_args(rest)
    tr, par = job.training, job.parallelism
    device = get_local_device()
    rank, _, world = dist_utils.world_info()
    world = dist_utils.init_distributed(job.comm, device, dump_folder=job.dump_folder)
    pdims = ParallelDims.from_config(par, world, rank).build()
    seed = job.debug.seed or 0
    torch.manual_seed(seed)                      # every rank builds the same initial weights
    cfg = hf_config(own.hf_model)
    model = HFCausalLM(cfg)
    if own.load_weights:
        from safetensors.torch import load_file

        state = {}
        for fn in sorted(f for f in os.listdir(own.hf_model) if f.endswith(".safetensors")):
            state.update(load_file(os.path.join(own.hf_model, fn)))
        missing, unexpected = model.hf.load_state_dict(state, strict=False)
        logger.info(f"loaded {len(state)} tensors ({len(missing)} missing, {len(unexpected)} unexpected)")
    if own.native_moe:
        from .moe_replacement import swap_native_moe

        logger.info(f"native MoE layer installed in {swap_native_moe(model)} decoder layers")
    n_params = sum(p.numel() for p in model.parameters())
    tokens, ctx = tr.num_tokens_per_microbatch_per_dp_rank, min(tr.max_context_length, tr.num_tokens_per_microbatch_per_dp_rank)
    data = _synthetic(cfg.vocab_size, tokens, ctx, seed * 1000 + pdims.dp_rank)
    if job.dataloader.dataset not in ("synthetic", "synthetic_mm"):
        tok = job.tokenizer.build(tokenizer_path=job.hf_assets_path)
        loader = job.dataloader.build(dp_world_size=pdims.dp_degree, dp_rank=pdims.dp_rank, num_tokens_per_batch=tokens,
                                      max_context_length=ctx, vocab_size=cfg.vocab_size, tokenizer=tok)
        data = ((b["input"], b["positions"], lab) for b, lab in loader)
    batches = [next(data) for _ in range(own.steps)] if pdims.pp_enabled else None
    t0 = time.perf_counter()
    if pdims.pp_enabled:
        schedule, engine, first, last = pipeline_hf(model, pdims=pdims, job_config=job, device=device, seed=seed)
        losses = hf_pipeline_train_steps(schedule, engine, batches, pdims=pdims, has_first=first, has_last=last,
                                         lr=job.optimizer.lr, max_norm=tr.max_norm)
    else:
        engine = parallelize_hf(model, pdims=pdims, job_config=job, device=device, seed=seed)
        opt = OptimizersContainer(job.optimizer, engines=[engine])
        sched = job.lr_scheduler.build(optimizers=opt, training_steps=own.steps)
        group = pdims.group("loss") if dist.is_initialized() and pdims.dp_degree > 1 else None
        losses = []
        for step in range(1, own.steps + 1):
            toks, pos, lab = (t.to(device) for t in next(data))
            n = (lab != -100).sum().float()
            if group is not None:
                dist.all_reduce(n, group=group)
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(toks, pos).float(), lab, ignore_index=-100, reduction="sum") / n
            loss.backward()
            engine.finish_backward()
            norm = clip_grad_norm_([engine], tr.max_norm, pdims, optimizers=opt)
            opt.step()
            sched.step()
            val = loss.detach().clone()
            if group is not None:
                dist.all_reduce(val, group=group)
            losses.append(float(val))
            if rank == 0 and step % max(job.metrics.log_freq, 1) == 0:
                logger.info(f"step {step:3d}  loss {losses[-1]:.4f}  grad norm {float(norm):.3f}")
    dt = time.perf_counter() - t0
    if rank == 0:
        logger.info(f"{type(model.hf).__name__}: {n_params / 1e6:.1f} M parameters, {own.steps} steps in {dt:.1f} s "
                    f"({own.steps * tokens * pdims.dp_degree / dt:.0f} tokens/s), loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    return losses


if __name__ == "__main__":
    init_logger()
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
