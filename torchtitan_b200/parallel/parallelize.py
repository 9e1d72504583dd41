"""Apply the parallelism plan to a decoder that is still on the meta device.

Order (parity with torchtitan/models/llama3/parallelize.py:23-80): tensor/sequence
parallel slicing of the weights -> context-parallel attention context -> expert
parallel slicing -> activation checkpointing -> sharded data parallelism (units =
embedding, every block, final norm + lm_head).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from torchtitan_b200.models.common.layers import TPContext
from torchtitan_b200.utils.logging import logger

from .activation_checkpoint import apply_activation_checkpointing
from .fsdp import ShardedModel, UnitSpec

__all__ = ["parallelize_decoder", "apply_tensor_parallel", "decoder_units"]


def apply_tensor_parallel(model: nn.Module, pdims, parallelism) -> TPContext | None:
    if not pdims.tp_enabled:
        return None
    if getattr(model, "mtp_layers", None) is not None:
        raise NotImplementedError("multi-token prediction layers are not tensor-parallel")
    tp = TPContext(group=pdims.group("tp"), size=pdims.tp, rank=pdims.local_rank("tp"),
                   sequence_parallel=parallelism.enable_sequence_parallel, comm=parallelism.tp_comm)
    if parallelism.tp_comm == "nvlink" and torch.cuda.is_available() and tp.sequence_parallel:
        # async tensor parallelism: the all-gather / reduce-scatter run inside the GEMM kernels
        from .symm import symm_available
        from .tp_fused import FusedTP

        if symm_available():
            dev = torch.device("cuda", torch.cuda.current_device())
            tp.fused = FusedTP(tp.group, dev, nbytes=int(parallelism.tp_symm_bytes))
    if model.tok_embeddings is not None:
        model.tok_embeddings.shard_(tp)
    for blk in model.layers.values():
        blk.attention.shard_(tp)
        if blk.feed_forward is not None:
            blk.feed_forward.shard_(tp)
        if blk.moe is not None:
            blk.moe.shard_tp_(tp)
        blk.tp = tp
    if model.lm_head is not None:
        model.lm_head.shard_("colwise", tp)
    model.tp = tp
    return tp


def decoder_units(model: nn.Module, pdims) -> list[UnitSpec]:
    units: list[UnitSpec] = []
    tied = getattr(model.config, "enable_weight_tying", False)
    if model.tok_embeddings is not None and not tied:
        units.append(UnitSpec("tok_embeddings", [model.tok_embeddings]))
    for name, blk in model.layers.items():
        if blk.moe is not None and pdims.ep_enabled:
            is_expert = lambda fqn, p: bool(getattr(p, "_is_expert", False))
            units.append(UnitSpec(f"layers.{name}.experts", [blk], group_name="efsdp", param_filter=is_expert))
            units.append(UnitSpec(f"layers.{name}", [blk], param_filter=lambda fqn, p: not getattr(p, "_is_expert", False)))
        else:
            units.append(UnitSpec(f"layers.{name}", [blk]))
    if getattr(model, "vision_encoder", None) is not None:
        units.append(UnitSpec("vision_encoder", [model.vision_encoder]))
    for name, blk in (getattr(model, "mtp_layers", None) or {}).items():
        if blk.moe is not None and pdims.ep_enabled:
            is_expert = lambda fqn, p: bool(getattr(p, "_is_expert", False))
            units.append(UnitSpec(f"mtp_layers.{name}.experts", [blk], group_name="efsdp", param_filter=is_expert))
            units.append(UnitSpec(f"mtp_layers.{name}", [blk], param_filter=lambda fqn, p: not getattr(p, "_is_expert", False)))
        else:
            units.append(UnitSpec(f"mtp_layers.{name}", [blk]))
    tail = [m for m in ((model.tok_embeddings if tied else None), model.norm, model.lm_head) if m is not None]
    if tail:
        units.append(UnitSpec("output", tail))
    return units


def parallelize_decoder(model: nn.Module, *, pdims, job_config, device: torch.device, seed: int = 0,
                        grad_accum_steps: int = 1, fqn_prefix: str = "", materialize: bool = True) -> ShardedModel:
    par = job_config.parallelism
    tr = job_config.training
    if pdims.ep_enabled:
        from .expert_parallel import apply_expert_parallel

        par._tokens_per_rank = tr.num_tokens_per_microbatch_per_dp_rank // max(1, pdims.tp * pdims.cp)
        apply_expert_parallel(model, pdims, par)
    tp = apply_tensor_parallel(model, pdims, par)
    if tp is not None or pdims.ep_enabled:
        # the slices the modules hold must be the ones their declared contracts name
        from . import sharding as shd

        if tp is not None:
            shd.check_against_slices(model, "tp")
        logger.debug("sharding contracts: %s", shd.sharding_table(model))

    if pdims.cp_enabled:
        from .context_parallel import CPContext

        model.cp = CPContext(group=pdims.group("cp"), size=pdims.cp, rank=pdims.local_rank("cp"),
                             mode=par.cp_comm, load_balancer=par.context_parallel_load_balancer or "none")
        if getattr(par, "cp_transport", "nccl") == "nvlink" and device.type == "cuda":
            from .cp_nvlink import CPNvlink
            from .symm import symm_available

            if symm_available():
                model.cp.nvlink = CPNvlink(model.cp.group, device, nbytes=int(par.cp_symm_bytes))
    apply_activation_checkpointing(model, job_config.activation_checkpoint)

    param_dtype = torch.bfloat16 if tr.mixed_precision_param == "bfloat16" else torch.float32
    if device.type == "cpu" and tr.dtype == "float32" and tr.mixed_precision_param == "float32":
        param_dtype = torch.float32
    state_dtype = torch.float32
    impl = getattr(job_config.optimizer, "implementation", "fused")
    if impl == "fused_opt_states_bf16":
        state_dtype = torch.bfloat16
    engine = ShardedModel(
        model, decoder_units(model, pdims), pdims=pdims, device=device, param_dtype=param_dtype,
        state_dtype=state_dtype, seed=seed, comm=par.fsdp_comm, grad_accum_steps=grad_accum_steps,
        fqn_prefix=fqn_prefix, tp=tp, offload_optimizer=bool(getattr(tr, "enable_cpu_offload", False)),
        reshard_after_forward=getattr(par, "fsdp_reshard_after_forward", "never") or "never",
    )
    if materialize:
        engine.materialize()
        hooks = []
        by_name = {u.name: u for u in engine.units}
        if model.tok_embeddings is not None:
            # the embedding's forward hook: waits for the optimizer step that refreshes it and, in the sharded layout,
            # gathers it before the lookup (it sits in the output unit when tied)
            emb_unit = by_name.get("tok_embeddings") or by_name.get("output")
            if emb_unit is not None:
                hooks.append((emb_unit, model.tok_embeddings))
        for name, blk in model.layers.items():
            for key in (f"layers.{name}", f"layers.{name}.experts"):
                if key in by_name:
                    hooks.append((by_name[key], blk))
        if "vision_encoder" in by_name:
            hooks.append((by_name["vision_encoder"], model.vision_encoder))
        for name, blk in (getattr(model, "mtp_layers", None) or {}).items():
            for key in (f"mtp_layers.{name}", f"mtp_layers.{name}.experts"):
                if key in by_name:
                    hooks.append((by_name[key], blk))
        if "output" in by_name and model.norm is not None:
            hooks.append((by_name["output"], model.norm))
        engine.attach_hooks(hooks)
    return engine
