"""Pipeline parallelism on ``torch.distributed.pipelining`` schedules with NCCL p2p.

Stage construction (parity: torchtitan/distributed/pipeline_parallel.py:65-640):

* the number of virtual stages is 1 per rank for single-stage schedules (GPipe, 1F1B), 2 per
  rank for looped / V schedules, or derived from ``pipeline_parallel_layers_per_stage``;
* layers are assigned with the embedding counted as ``first_stage_less_layers`` and
  norm + lm_head as ``last_stage_less_layers`` extra "layers": ``eff = L + in + out``,
  ``base = eff // S``, the first ``eff % S`` stages get one more;
* rank r owns stages ``{r, r+pp, ...}`` (loop) or ``{r, 2pp-1-r}`` (V style for ZBV/DualPipeV);
* every stage is a pruned deep copy of the meta model (layer names keep their index, so FQNs
  are stable), parallelised by the model's own ``parallelize_fn`` and wrapped in its own
  sharded engine.

Microbatches use the folded-token layout: the schedule chunks ``[n_mb, T]`` inputs along dim 0
and the stage wrapper removes / restores that unit dimension.  Gradients of a stage are
accumulated locally over the microbatches of a step and reduced once (``scale_grads=False``:
the loss is already divided by the global token count).
"""

from __future__ import annotations

import copy

import torch
import torch.nn as nn

from torchtitan_b200.components.loss import LinearCrossEntropyLoss
from torchtitan_b200.utils.logging import logger

__all__ = ["pipeline_decoder", "stage_layer_assignment", "stage_ids_for_rank", "run_pipeline_step",
           "run_pipeline_eval", "num_virtual_stages"]

_V_SCHEDULES = ("ZBVZeroBubble", "DualPipeV")
_SINGLE = ("GPipe", "1F1B")


def num_virtual_stages(parallelism, n_layers: int, pp: int) -> int:
    sched = parallelism.pipeline_parallel_schedule
    lps = parallelism.pipeline_parallel_layers_per_stage
    if lps is not None:
        eff = n_layers + parallelism.pipeline_parallel_first_stage_less_layers + \
            parallelism.pipeline_parallel_last_stage_less_layers
        total = -(-eff // lps)
        if total % pp:
            raise ValueError(f"{total} stages (layers_per_stage={lps}) cannot be spread evenly over pp={pp}")
        per_rank = total // pp
        if sched in _SINGLE and per_rank != 1:
            raise ValueError(f"schedule {sched} needs exactly one stage per rank, got {per_rank}")
        if sched in _V_SCHEDULES and per_rank != 2:
            raise ValueError(f"schedule {sched} needs exactly two stages per rank, got {per_rank}")
        return total
    return pp if sched in _SINGLE else 2 * pp


def stage_layer_assignment(n_layers: int, num_stages: int, input_weight: int = 1, output_weight: int = 1):
    """``[(has_embedding, [layer ids], has_output)]`` per stage."""
    eff = n_layers + input_weight + output_weight
    if num_stages > eff:
        raise ValueError(f"{num_stages} stages for {eff} effective layers")
    base, extra = divmod(eff, num_stages)
    out, nxt = [], 0
    for s in range(num_stages):
        quota = base + (1 if s < extra else 0)
        first, last = s == 0, s == num_stages - 1
        n = quota - (input_weight if first else 0) - (output_weight if last else 0)
        if num_stages == 1:
            n = n_layers
        if n < 0:
            raise ValueError("stage weights leave a stage with a negative number of layers")
        if last:
            n = n_layers - nxt
        out.append((first, list(range(nxt, nxt + n)), last))
        nxt += n
    return out


def stage_ids_for_rank(pp_rank: int, pp: int, num_stages: int, style: str = "loop") -> list[int]:
    per = num_stages // pp
    if style == "v":
        assert per == 2, "V-style schedules use two stages per rank"
        return [pp_rank, num_stages - 1 - pp_rank]
    return [pp_rank + i * pp for i in range(per)]


def _prune(model: nn.Module, has_emb: bool, layer_ids: list[int], has_out: bool, fqns: list[str] | None = None):
    part = copy.deepcopy(model)
    # Parameter.__deepcopy__ drops python attributes: carry the init / sharding annotations over
    for (_, old), (_, new) in zip(model.named_parameters(remove_duplicate=False),
                                  part.named_parameters(remove_duplicate=False)):
        for attr in ("_init_spec", "_tp_slices", "_replicated_over_tp", "_is_expert"):
            if hasattr(old, attr):
                setattr(new, attr, getattr(old, attr))
    keep = {str(i) for i in layer_ids}
    if fqns is not None:
        has_emb = "tok_embeddings" in fqns
        has_out = "lm_head" in fqns or "norm" in fqns
        keep = {f.split(".")[1] for f in fqns if f.startswith("layers.")}
    if not has_emb:
        part.tok_embeddings = None
    for name in list(part.layers.keys()):
        if name not in keep:
            del part.layers[name]
    if not has_out:
        part.norm = None
        part.lm_head = None
    return part


class _StageModule(nn.Module):
    """Adapts a decoder part to the schedule's calling convention (unit leading dim)."""

    def __init__(self, part: nn.Module, is_last: bool):
        super().__init__()
        self.part = part
        self.is_last = is_last

    def forward(self, x, positions=None, q_pos=None):
        x = x.squeeze(0)
        pos = positions.squeeze(0) if positions is not None else None
        qp = q_pos.squeeze(0) if q_pos is not None else None
        ctx = self.part.build_context(pos, qp) if pos is not None else None
        h = self.part(x, pos, ctx, return_hidden=True)
        return h.unsqueeze(0)


class _PipelineLoss:
    """Loss on the last stage: fused lm_head + CE on the stage output (final hidden states)."""

    def __init__(self, loss_fn):
        self.loss_fn = loss_fn
        self.global_valid: torch.Tensor | float = 1.0

    def __call__(self, output, target):
        return self.loss_fn(output.squeeze(0), target.squeeze(0), self.global_valid)


def pipeline_decoder(model: nn.Module, *, pdims, job_config, device, seed, parallelize_fn, loss_fn,
                     grad_accum_steps: int = 1):
    from torch.distributed.pipelining import PipelineStage
    from torch.distributed.pipelining.schedules import PipelineScheduleSingle, get_schedule_class

    par = job_config.parallelism
    pp, pp_rank = pdims.pp, pdims.local_rank("pp")
    if getattr(model.config, "enable_weight_tying", False):
        raise ValueError("weight tying between embedding and lm_head is not supported with pipeline parallelism")
    n_layers = len(model.layers)
    sched_name = par.pipeline_parallel_schedule
    sched_cls = get_schedule_class(sched_name)
    fqn_parts = par.module_fqns_per_model_part
    if fqn_parts:
        num_stages = len(fqn_parts)
        assign = [(False, [], False)] * num_stages
    else:
        num_stages = num_virtual_stages(par, n_layers, pp)
        assign = stage_layer_assignment(n_layers, num_stages, par.pipeline_parallel_first_stage_less_layers,
                                        par.pipeline_parallel_last_stage_less_layers)
    style = "v" if sched_name in _V_SCHEDULES else "loop"
    mine = stage_ids_for_rank(pp_rank, pp, num_stages, style)
    n_mb = par.num_pp_microbatches
    if n_mb < pp:
        logger.warning(f"num_pp_microbatches ({n_mb}) < pipeline degree ({pp}): the pipeline will have bubbles")

    stages, parts, engines = [], [], []
    for sid in mine:
        has_emb, layer_ids, has_out = assign[sid]
        part = _prune(model, has_emb, layer_ids, has_out, fqn_parts[sid] if fqn_parts else None)
        engine = parallelize_fn(part, pdims=pdims, job_config=job_config, device=device, seed=seed,
                                grad_accum_steps=max(2, grad_accum_steps))
        engine.defer_reduce = True
        wrapped = _StageModule(part, sid == num_stages - 1)
        stages.append(PipelineStage(wrapped, sid, num_stages, device, group=pdims.group("pp")))
        parts.append(part)
        engines.append(engine)
        logger.info(f"PP rank {pp_rank} builds stage {sid}: embedding={part.tok_embeddings is not None} "
                    f"layers={list(part.layers.keys())} output={part.lm_head is not None}")
    has_first = 0 in mine
    has_last = (num_stages - 1) in mine
    ploss = _PipelineLoss(loss_fn)
    if has_last and isinstance(loss_fn, LinearCrossEntropyLoss):
        last_part = parts[mine.index(num_stages - 1)]
        loss_fn.set_lm_head(last_part.lm_head, tp=last_part.tp)
    if issubclass(sched_cls, PipelineScheduleSingle):
        if len(stages) != 1:
            raise ValueError(f"schedule {sched_name} supports one stage per rank")
        schedule = sched_cls(stages[0], n_microbatches=n_mb, loss_fn=ploss, scale_grads=False)
    else:
        schedule = sched_cls(stages, n_microbatches=n_mb, loss_fn=ploss, scale_grads=False)
        csv = par.pipeline_parallel_schedule_csv
        if csv:
            schedule._load_csv(csv)
    schedule._tb200_loss = ploss
    logger.info(f"Using pipeline schedule {sched_name} with {n_mb} microbatches and {num_stages} stages")
    return schedule, parts, engines, has_first, has_last


def run_pipeline_step(trainer, tokens, positions, labels, q_pos, global_valid) -> torch.Tensor:
    """One forward/backward over all microbatches; returns the summed loss (zero off the last stage)."""
    sched = trainer.pp_schedule
    sched._tb200_loss.global_valid = global_valid
    kwargs = {"positions": positions}
    if q_pos is not None:
        kwargs["q_pos"] = q_pos.unsqueeze(0).expand(tokens.shape[0], -1).contiguous()
    losses: list[torch.Tensor] = []
    target = labels if trainer.pp_has_last_stage else None
    if trainer.pp_has_first_stage:
        sched.step(tokens, target=target, losses=losses, return_outputs=False, **kwargs)
    else:
        sched.step(target=target, losses=losses, return_outputs=False, **kwargs)
    for e in trainer.engines:
        e.finish_backward(flush=True)
    if trainer.pp_has_last_stage and losses:
        return torch.stack([l.detach().reshape(()) for l in losses]).sum()
    return torch.zeros((), dtype=torch.float32, device=trainer.device)


@torch.no_grad()
def run_pipeline_eval(trainer, tokens, positions, labels, q_pos) -> torch.Tensor:
    sched = trainer.pp_schedule
    sched._tb200_loss.global_valid = 1.0
    if tokens.dim() == 1:
        tokens, positions, labels = tokens.unsqueeze(0), positions.unsqueeze(0), labels.unsqueeze(0)
    kwargs = {"positions": positions}
    losses: list[torch.Tensor] = []
    target = labels if trainer.pp_has_last_stage else None
    if trainer.pp_has_first_stage:
        sched.eval(tokens, target=target, losses=losses, **kwargs)
    else:
        sched.eval(target=target, losses=losses, **kwargs)
    if trainer.pp_has_last_stage and losses:
        return torch.stack([l.detach().reshape(()) for l in losses]).sum()
    return torch.zeros((), dtype=torch.float32, device=trainer.device)
