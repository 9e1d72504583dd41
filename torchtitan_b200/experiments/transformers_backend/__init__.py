"""Train Hugging Face ``transformers`` causal-LM architectures with this framework's folded-token
interface, loss and data pipeline (parity: torchtitan/experiments/transformers_modeling_backend).

``HFCausalLM(config_or_name)`` builds the architecture from a ``transformers`` config (random
init) and exposes ``forward(tokens[T], positions[T]) -> logits[T, V]``; documents are kept apart by
passing ``position_ids`` that restart per document together with a block-diagonal causal mask.
``hf_train_steps`` is a minimal data-parallel loop (gradient averaging over the world group), the oracle of the
tests.  ``parallelize_hf`` puts the same module under this framework's sharded data-parallel engine (units =
embedding, every decoder layer, final norm + lm_head; resident or sharded parameter layout, NCCL or NVLink
transport, fp32 master weights and sharded AdamW: parity with parallelize.py of the reference's backend, which
applies FSDP to the HF layers), and ``hf_engine_train_steps`` is the training loop on it.  With a tensor-parallel
degree in ``pdims`` the attention and MLP projections of every decoder layer are split first (``apply_hf_tensor_parallel``:
q / k / v / gate / up column-wise, o / down row-wise with an all-reduce, activations replicated between the layers;
parity: hf_sharding.py of the reference's backend).  ``pipeline_hf`` splits the decoder layers over the pipeline
ranks (one stage per rank, GPipe / 1F1B, every stage under the sharded engine) and ``hf_pipeline_train_steps`` trains
on the schedule."""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ["HFCausalLM", "hf_train_steps", "parallelize_hf", "hf_engine_train_steps", "apply_hf_tensor_parallel",
           "pipeline_hf", "hf_pipeline_train_steps"]


class HFCausalLM(nn.Module):
    def __init__(self, config, *, attn_implementation: str = "sdpa", dtype=torch.float32):
        super().__init__()
        from transformers import AutoConfig, AutoModelForCausalLM

        if isinstance(config, str):
            config = AutoConfig.from_pretrained(config)
        config._attn_implementation = attn_implementation
        self.hf = AutoModelForCausalLM.from_config(config).to(dtype)
        self.vocab_size = config.vocab_size

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        T = tokens.shape[0]
        if positions is None:
            positions = torch.arange(T, device=tokens.device)
        doc = torch.cumsum((positions == 0).long(), 0)
        allowed = (doc[:, None] == doc[None, :]) & torch.ones(T, T, dtype=torch.bool, device=tokens.device).tril()
        mask = torch.zeros(T, T, device=tokens.device, dtype=self.hf.dtype).masked_fill(~allowed, torch.finfo(self.hf.dtype).min)
        out = self.hf(input_ids=tokens[None], position_ids=positions[None], attention_mask=mask[None, None])
        return out.logits[0]


def hf_train_steps(model: HFCausalLM, batches, *, lr: float = 3e-4, max_norm: float = 1.0) -> list[float]:
    """``batches``: iterable of ``(tokens[T], positions[T], labels[T])``; returns the per-step losses."""
    opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1)
    losses = []
    for tokens, positions, labels in batches:
        logits = model(tokens, positions)
        loss = nn.functional.cross_entropy(logits.float(), labels, ignore_index=-100)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        if dist.is_initialized() and dist.get_world_size() > 1:
            for p in model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm)
        opt.step()
        losses.append(float(loss.detach()))
    return losses


_COLWISE = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
_ROWWISE = ("o_proj", "down_proj")


class _TPLinear(nn.Module):
    """A projection of an HF layer split over the tensor-parallel group.  ``colwise``: this rank's output features,
    the (replicated) input passes through an identity whose backward sums the input gradient over the group.
    ``rowwise``: this rank's input features, the partial products are summed with an all-reduce, the bias added once."""

    def __init__(self, lin: nn.Linear, mode: str, tp):
        super().__init__()
        self.mode, self.tp = mode, tp
        out_f, in_f = lin.weight.shape
        dim = 0 if mode == "colwise" else 1
        full = out_f if dim == 0 else in_f
        if full % tp.size:
            raise ValueError(f"{mode} projection of {full} features does not divide by tp={tp.size}")
        n = full // tp.size
        lo, hi = tp.rank * n, (tp.rank + 1) * n
        w = lin.weight.detach()[lo:hi] if dim == 0 else lin.weight.detach()[:, lo:hi]
        self.weight = nn.Parameter(w.clone().contiguous())
        self.weight._tp_slices = (dim, [(lo, hi)], (out_f, in_f))
        self.bias = None
        if lin.bias is not None:
            if dim == 0:
                self.bias = nn.Parameter(lin.bias.detach()[lo:hi].clone())
                self.bias._tp_slices = (0, [(lo, hi)], (out_f,))
            else:
                self.bias = nn.Parameter(lin.bias.detach().clone())
                self.bias._replicated_over_tp = True
                self.bias._tp_grad_complete_without_sp = True

    def forward(self, x):
        from torchtitan_b200.parallel import tp_ops

        if self.mode == "colwise":
            return nn.functional.linear(tp_ops.copy_to_tp(x, self.tp), self.weight, self.bias)
        y = tp_ops.all_reduce(nn.functional.linear(x, self.weight), self.tp)
        return y if self.bias is None else y + self.bias


def apply_hf_tensor_parallel(model: HFCausalLM, tp) -> int:
    """Split the attention / MLP projections of every decoder layer over ``tp`` (a ``TPContext`` with
    ``sequence_parallel = False``); every other parameter stays replicated.  Returns the number of projections split."""
    if tp.sequence_parallel:
        raise ValueError("HF modules run with replicated activations: build the TPContext with sequence_parallel=False")
    n = 0
    inside = set()
    for layer in model.hf.model.layers:
        for parent in layer.modules():
            for name, child in list(parent.named_children()):
                if isinstance(child, nn.Linear) and name in _COLWISE + _ROWWISE:
                    setattr(parent, name, _TPLinear(child, "colwise" if name in _COLWISE else "rowwise", tp))
                    n += 1
        attn = getattr(layer, "self_attn", None)
        if attn is not None:
            # per-head norms (q_norm / k_norm) act on this rank's heads: their gradients are per-rank parts
            inside.update(id(p) for name, m in attn.named_children() if "norm" in name for p in m.parameters())
    for p in model.parameters():
        if getattr(p, "_tp_slices", None) is None:
            p._replicated_over_tp = True
            if id(p) not in inside:
                p._tp_grad_complete_without_sp = True    # seen after the all-reduce: complete on every rank
    return n


def _hf_units(model: HFCausalLM):
    from torchtitan_b200.parallel.fsdp import UnitSpec

    base = model.hf.model
    layers = list(base.layers)
    tied = model.hf.lm_head.weight is base.embed_tokens.weight
    units, hooks = [], []
    if not tied:
        units.append(UnitSpec("embed_tokens", [base.embed_tokens]))
        hooks.append(("embed_tokens", base.embed_tokens))
    for i, layer in enumerate(layers):
        units.append(UnitSpec(f"layers.{i}", [layer]))
        hooks.append((f"layers.{i}", layer))
    tail = ([base.embed_tokens] if tied else []) + [base.norm, model.hf.lm_head]
    units.append(UnitSpec("output", tail))
    hooks.append(("output", base.embed_tokens if tied else base.norm))
    if tied:
        hooks.append(("output", base.norm))
    rest = [m for n, m in base.named_children() if n not in ("embed_tokens", "layers", "norm")]
    if any(True for m in rest for _ in m.parameters()):
        units.append(UnitSpec("extras", rest))
    return units, hooks


def parallelize_hf(model: HFCausalLM, *, pdims, job_config, device: torch.device, seed: int = 0):
    """Shard an ``HFCausalLM`` with the flat-buffer engine, keeping the values the HF initialiser gave it."""
    from torchtitan_b200.parallel.fsdp import ShardedModel

    par, tr = job_config.parallelism, job_config.training
    tp = None
    if pdims.tp_enabled:
        from torchtitan_b200.models.common.layers import TPContext

        tp = TPContext(group=pdims.group("tp"), size=pdims.tp, rank=pdims.local_rank("tp"), sequence_parallel=False)
        apply_hf_tensor_parallel(model, tp)
    values = {n: p.detach().float().cpu().clone() for n, p in model.named_parameters()}
    units, hooks = _hf_units(model)
    param_dtype = torch.bfloat16 if tr.mixed_precision_param == "bfloat16" else torch.float32
    engine = ShardedModel(model, units, pdims=pdims, device=device, param_dtype=param_dtype, seed=seed, tp=tp,
                          comm=par.fsdp_comm, reshard_after_forward=par.fsdp_reshard_after_forward or "never")
    model.to(device)          # buffers (rotary tables); parameters are replaced by views of the flat buffers below
    engine.materialize(init=False)
    with torch.no_grad():
        for u in engine.units:
            for slot, pstart, sstart, n in u.slot_pieces():
                u.master[sstart:sstart + n].copy_(values[slot.fqn].reshape(-1)[pstart:pstart + n])
    engine.publish_params()
    by_name = {u.name: u for u in engine.units}
    engine.attach_hooks([(by_name[name], module) for name, module in hooks if name in by_name])
    return engine


def hf_engine_train_steps(model: HFCausalLM, engine, batches, *, pdims, lr: float = 3e-4, max_norm: float = 1.0) -> list[float]:
    """Like ``hf_train_steps`` on the sharded engine: the loss is divided by the global token count, gradients are
    reduce-scattered per unit during backward, AdamW runs on the fp32 shards."""
    from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_

    opt = OptimizersContainer(OptimizersContainer.Config(lr=lr), engines=[engine])
    losses = []
    # token counts and losses are summed over the ranks that hold different data (tensor-parallel ranks share a batch)
    loss_group = pdims.group("loss") if (dist.is_initialized() and pdims.world_size > 1 and pdims.dp_degree > 1) else None
    for tokens, positions, labels in batches:
        dev = engine.device
        tokens, positions, labels = tokens.to(dev), positions.to(dev), labels.to(dev)
        n = (labels != -100).sum().float()
        if loss_group is not None:
            dist.all_reduce(n, group=loss_group)
        opt.zero_grad()
        logits = model(tokens, positions)
        loss = nn.functional.cross_entropy(logits.float(), labels, ignore_index=-100, reduction="sum") / n
        loss.backward()
        engine.finish_backward()
        clip_grad_norm_([engine], max_norm, pdims, optimizers=opt)
        opt.step()
        losses.append(loss.detach())
    out = torch.stack(losses)
    if loss_group is not None:
        dist.all_reduce(out, group=loss_group)
    return out.tolist()


# ---------------------------------------------------------------------------------------------------------------
# pipeline parallelism for HF decoder stacks


class _HFStage(nn.Module):
    """A contiguous slice of an HF decoder stack in the schedule's calling convention: ``x`` is ``[1, T]`` token ids
    on the first stage and ``[1, T, D]`` hidden states elsewhere; ``positions [1, T]`` reach every stage as a keyword
    argument, so each stage derives its own rotary tables and per-document causal mask."""

    def __init__(self, hf, layer_ids: list[int], first: bool, last: bool):
        super().__init__()
        base = hf.model
        self.embed_tokens = base.embed_tokens if first else None
        self.layers = nn.ModuleList([base.layers[i] for i in layer_ids])
        self.rotary_emb = base.rotary_emb
        self.norm = base.norm if last else None
        self.lm_head = hf.lm_head if last else None

    def forward(self, x, positions=None):
        T = x.shape[1]
        if positions is None:
            positions = torch.arange(T, device=x.device)[None]
        h = self.embed_tokens(x) if self.embed_tokens is not None else x
        pos = positions[0]
        doc = torch.cumsum((pos == 0).long(), 0)
        allowed = (doc[:, None] == doc[None, :]) & torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
        mask = torch.zeros(T, T, device=x.device, dtype=h.dtype).masked_fill(~allowed, torch.finfo(h.dtype).min)
        cos_sin = self.rotary_emb(h, positions)
        for layer in self.layers:
            out = layer(h, attention_mask=mask[None, None], position_ids=positions, position_embeddings=cos_sin)
            h = out[0] if isinstance(out, tuple) else out
        if self.norm is not None:
            h = self.lm_head(self.norm(h))
        return h


class _HFPipelineLoss:
    def __init__(self):
        self.global_valid: torch.Tensor | float = 1.0

    def __call__(self, logits, target):
        return nn.functional.cross_entropy(logits[0].float(), target[0], ignore_index=-100, reduction="sum") / self.global_valid


def pipeline_hf(model: HFCausalLM, *, pdims, job_config, device: torch.device, seed: int = 0):
    """Split the decoder layers of an ``HFCausalLM`` over the pipeline ranks (embedding on the first stage, final
    norm + lm_head on the last; parity: pipeline.py of the reference's backend) and put every stage under the sharded
    engine.  Returns ``(schedule, stage module, engine, has_first, has_last)``; single-stage-per-rank schedules
    (GPipe, 1F1B)."""
    from torch.distributed.pipelining import PipelineStage
    from torch.distributed.pipelining.schedules import PipelineScheduleSingle, get_schedule_class

    from torchtitan_b200.parallel.fsdp import ShardedModel, UnitSpec
    from torchtitan_b200.parallel.pipeline import stage_layer_assignment

    par, tr = job_config.parallelism, job_config.training
    if model.hf.lm_head.weight is model.hf.model.embed_tokens.weight:
        raise ValueError("tied embeddings span the first and the last pipeline stage: not supported")
    sched_cls = get_schedule_class(par.pipeline_parallel_schedule)
    if not issubclass(sched_cls, PipelineScheduleSingle):
        raise ValueError("the HF pipeline plan runs one stage per rank (GPipe or 1F1B)")
    pp, sid = pdims.pp, pdims.local_rank("pp")
    first, layer_ids, last = stage_layer_assignment(len(model.hf.model.layers), pp)[sid]
    stage = _HFStage(model.hf, layer_ids, first, last)
    values = {n: p.detach().float().cpu().clone() for n, p in stage.named_parameters()}
    units, hooks = [], []
    if first:
        units.append(UnitSpec("embed_tokens", [stage.embed_tokens]))
        hooks.append(("embed_tokens", stage.embed_tokens))
    for i, layer in zip(layer_ids, stage.layers):
        units.append(UnitSpec(f"layers.{i}", [layer]))
        hooks.append((f"layers.{i}", layer))
    if last:
        units.append(UnitSpec("output", [stage.norm, stage.lm_head]))
        hooks.append(("output", stage.norm))
    param_dtype = torch.bfloat16 if tr.mixed_precision_param == "bfloat16" else torch.float32
    engine = ShardedModel(stage, units, pdims=pdims, device=device, param_dtype=param_dtype, seed=seed,
                          comm=par.fsdp_comm, reshard_after_forward="never", grad_accum_steps=2)
    engine.defer_reduce = True        # gradients accumulate over the microbatches, one reduction per step
    stage.to(device)
    engine.materialize(init=False)
    with torch.no_grad():
        for u in engine.units:
            for slot, pstart, sstart, n in u.slot_pieces():
                u.master[sstart:sstart + n].copy_(values[slot.fqn].reshape(-1)[pstart:pstart + n])
    engine.publish_params()
    by_name = {u.name: u for u in engine.units}
    engine.attach_hooks([(by_name[name], module) for name, module in hooks])
    ploss = _HFPipelineLoss()
    pstage = PipelineStage(stage, sid, pp, device, group=pdims.group("pp"))
    schedule = sched_cls(pstage, n_microbatches=par.num_pp_microbatches, loss_fn=ploss, scale_grads=False)
    schedule._tb200_loss = ploss
    return schedule, stage, engine, first, last


def hf_pipeline_train_steps(schedule, engine, batches, *, pdims, has_first: bool, has_last: bool, lr: float = 3e-4,
                            max_norm: float = 1.0) -> list[float]:
    """``batches``: per step ``(tokens [M, T], positions [M, T], labels [M, T])`` with M microbatches.  Returns the
    per-step losses (summed over the pipeline group, so every rank returns them)."""
    from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_

    opt = OptimizersContainer(OptimizersContainer.Config(lr=lr), engines=[engine])
    dev = engine.device
    out = []
    loss_group = pdims.group("loss") if (pdims.dp_degree > 1) else None
    for tokens, positions, labels in batches:
        tokens, positions, labels = tokens.to(dev), positions.to(dev), labels.to(dev)
        n = (labels != -100).sum().float()
        if loss_group is not None:
            dist.all_reduce(n, group=loss_group)
        schedule._tb200_loss.global_valid = n
        opt.zero_grad()
        losses: list[torch.Tensor] = []
        target = labels if has_last else None
        if has_first:
            schedule.step(tokens, target=target, losses=losses, return_outputs=False, positions=positions)
        else:
            schedule.step(target=target, losses=losses, return_outputs=False, positions=positions)
        engine.finish_backward(flush=True)
        clip_grad_norm_([engine], max_norm, pdims, optimizers=opt)
        opt.step()
        step_loss = torch.stack([l.detach().reshape(()) for l in losses]).sum() if (has_last and losses) else \
            torch.zeros((), device=dev)
        out.append(step_loss)
    res = torch.stack(out)
    dist.all_reduce(res, group=pdims.group("pp"))       # only the last stage holds the loss
    if loss_group is not None:
        dist.all_reduce(res, group=loss_group)
    return res.tolist()
