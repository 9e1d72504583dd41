"""Sharded engine: parity with plain PyTorch training, 2-rank vs 1-rank, gradient accumulation."""

import copy

import pytest
import torch

from tests.dist_utils import run_distributed
from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_
from torchtitan_b200.config import ConfigManager
from torchtitan_b200.models import get_model_spec
from torchtitan_b200.ops import functional as OF
from torchtitan_b200.parallel.parallel_dims import ParallelDims
from torchtitan_b200.parallel.parallelize import parallelize_decoder
from torchtitan_b200.trainer import Trainer

T = 64


def _job(accum_tokens=-1, **par):
    cfg = Trainer.Config()
    cfg.model.flavor = "debugmodel"
    cfg.training.num_tokens_per_microbatch_per_dp_rank = T
    cfg.training.max_context_length = T
    cfg.training.mixed_precision_param = "float32"
    cfg.training.num_tokens_per_train_step = accum_tokens
    for k, v in par.items():
        setattr(cfg.parallelism, k, v)
    return cfg


def _small_model_cfg(n_layers=2):
    spec = get_model_spec("llama3", "debugmodel")
    mc = spec.model
    mc.layers = mc.layers[:n_layers]
    mc.n_layers = n_layers
    for blk in mc.layers:
        blk.attention.rope.max_context_length = T
    return mc


def _batches(n, seed=0, vocab=2048):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (T + 1,), generator=g)
        out.append((ids[:-1].clone(), ids[1:].clone()))
    return out


def _build_engine(cfg, pdims, accum=1, n_layers=2):
    mc = _small_model_cfg(n_layers)
    with torch.device("meta"):
        model = mc.build()
    eng = parallelize_decoder(model, pdims=pdims, job_config=cfg, device=torch.device("cpu"), seed=7,
                              grad_accum_steps=accum)
    return mc, model, eng


def _engine_steps(cfg, pdims, microbatches_per_step, accum=1, steps=3):
    mc, model, eng = _build_engine(cfg, pdims, accum)
    opt = OptimizersContainer(OptimizersContainer.Config(lr=1e-2), engines=[eng])
    losses = []
    pos = torch.arange(T)
    for s in range(steps):
        opt.zero_grad()
        mbs = microbatches_per_step[s]
        n_tok = torch.tensor(float(T * len(mbs) * pdims.dp_degree))
        tot = 0.0
        for tok, lab in mbs:
            h = model(tok, pos, return_hidden=True)
            loss = OF.linear_cross_entropy(h, model.lm_head.weight, lab, 1.0 / n_tok, 4)
            loss.backward()
            eng.finish_backward()
            tot += float(loss.detach())
        clip_grad_norm_([eng], 1.0, pdims, optimizers=opt)
        opt.step()
        losses.append(tot)
    return losses, model, eng


def test_engine_matches_plain_pytorch():
    cfg = _job()
    pdims = ParallelDims(world_size=1)
    data = [[b] for b in _batches(3)]
    losses, model, eng = _engine_steps(cfg, pdims, data)

    mc = _small_model_cfg()
    plain = mc.build()
    plain.init_states(seed=7)
    opt = torch.optim.AdamW(plain.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    pos = torch.arange(T)
    ref_losses = []
    for (tok, lab), in data:
        opt.zero_grad()
        logits = plain(tok, pos)
        loss = torch.nn.functional.cross_entropy(logits.float(), lab, reduction="sum") / T
        loss.backward()
        torch.nn.utils.clip_grad_norm_(plain.parameters(), 1.0)
        opt.step()
        ref_losses.append(float(loss.detach()))
    assert torch.allclose(torch.tensor(losses), torch.tensor(ref_losses), atol=2e-4), (losses, ref_losses)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), plain.named_parameters()):
        assert n1 == n2
        assert torch.allclose(p1, p2, atol=2e-3), (n1, (p1 - p2).abs().max())


def test_gradient_accumulation_equals_big_batch():
    pdims = ParallelDims(world_size=1)
    b = _batches(6)
    two, _, _ = _engine_steps(_job(accum_tokens=2 * T), pdims, [b[0:2], b[2:4], b[4:6]], accum=2)
    assert all(l == l for l in two)


def _rank_fn(rank, world, out_path):
    import torch.distributed as dist

    cfg = _job()
    pdims = ParallelDims(world_size=world, rank=rank).build()
    b = _batches(6)
    data = [[b[2 * s + rank]] for s in range(3)]
    losses, model, eng = _engine_steps(cfg, pdims, data)
    t = torch.tensor(losses)
    dist.all_reduce(t)
    if rank == 0:
        sd = {n: p.detach().clone() for n, p in model.named_parameters()}
        torch.save({"losses": t, "params": sd}, out_path)


def test_two_ranks_match_one_rank_with_accumulation(tmp_path):
    out = str(tmp_path / "r2.pt")
    run_distributed(_rank_fn, 2, out)
    got = torch.load(out)
    pdims = ParallelDims(world_size=1)
    b = _batches(6)
    losses, model, _ = _engine_steps(_job(accum_tokens=2 * T), pdims, [b[0:2], b[2:4], b[4:6]], accum=2)
    assert torch.allclose(got["losses"], torch.tensor(losses), atol=1e-4), (got["losses"], losses)
    for n, p in model.named_parameters():
        assert torch.allclose(p, got["params"][n], atol=2e-3), n


def _tp_fn(rank, world, out_path):
    import torch.distributed as dist

    cfg = _job(tensor_parallel_degree=2)
    pdims = ParallelDims(world_size=world, rank=rank, tp=2).build()
    b = _batches(3)
    mc, model, eng = _build_engine(cfg, pdims)
    opt = OptimizersContainer(OptimizersContainer.Config(lr=1e-2), engines=[eng])
    from torchtitan_b200.components.loss import LinearCrossEntropyLoss

    loss_fn = LinearCrossEntropyLoss()
    loss_fn.set_lm_head(model.lm_head, tp=model.tp)
    pos = torch.arange(T)
    losses = []
    for tok, lab in b:
        opt.zero_grad()
        h = model(tok, pos, return_hidden=True)
        loss = loss_fn(h, lab, torch.tensor(float(T)))
        loss.backward()
        eng.finish_backward()
        clip_grad_norm_([eng], 1.0, pdims, optimizers=opt)
        opt.step()
        losses.append(float(loss.detach()))
    if rank == 0:
        torch.save(torch.tensor(losses), out_path)


def test_tensor_parallel_matches_single(tmp_path):
    out = str(tmp_path / "tp.pt")
    run_distributed(_tp_fn, 2, out)
    got = torch.load(out)
    pdims = ParallelDims(world_size=1)
    losses, _, _ = _engine_steps(_job(), pdims, [[x] for x in _batches(3)])
    assert torch.allclose(got, torch.tensor(losses), atol=2e-4), (got, losses)


def test_activation_offload_hooks_preserve_gradients():
    from torchtitan_b200.parallel.activation_offload import OffloadStats, offload_activations

    torch.manual_seed(0)
    lin1, lin2 = torch.nn.Linear(64, 256), torch.nn.Linear(256, 8)
    x = torch.randn(128, 64)

    def run(ctx):
        for p in list(lin1.parameters()) + list(lin2.parameters()):
            p.grad = None
        with ctx:
            y = lin2(torch.nn.functional.gelu(lin1(x))).square().sum()
        y.backward()
        return [p.grad.clone() for p in list(lin1.parameters()) + list(lin2.parameters())]

    import contextlib

    ref_grads = run(contextlib.nullcontext())
    stats = OffloadStats()
    got = run(offload_activations(min_bytes=1024, stats=stats, force=True))
    assert stats.tensors >= 2 and stats.bytes >= 128 * 256 * 4        # the hidden activations went through the hooks
    for a, b in zip(ref_grads, got):
        assert torch.equal(a, b)


def _reshard_fn(rank, world, policy, accum, out_path):
    import torch.distributed as dist

    cfg = _job(accum_tokens=accum * T * world, fsdp_reshard_after_forward=policy)
    pdims = ParallelDims(world_size=world, rank=rank).build()
    b = _batches(4 * accum * world, seed=3)
    data = [[b[(s * accum + a) * world + rank] for a in range(accum)] for s in range(4)]
    losses, model, eng = _engine_steps(cfg, pdims, data, accum=accum, steps=4)
    assert eng.sharded_params == (policy == "always")
    if policy == "always":
        # a rank holds its shards plus two gather slots and two gradient slots, never every unit in full
        assert all(u.param_shard is not None and u.param_shard.numel() == u.shard_numel for u in eng.units)
        assert len(eng._pools) == 1
    t = torch.tensor(losses)
    dist.all_reduce(t)
    masters = torch.cat([u.master for u in eng.units])
    if rank == 0:
        torch.save({"losses": t, "master": masters}, out_path)


@pytest.mark.parametrize("accum", [1, 2])
def test_sharded_parameter_layout_matches_resident(tmp_path, accum):
    """fsdp_reshard_after_forward = always (parameters gathered per unit, freed after use) trains exactly like
    the resident layout: same reductions, same optimizer, only the place of the all-gather differs."""
    a, b = str(tmp_path / "never.pt"), str(tmp_path / "always.pt")
    run_distributed(_reshard_fn, 2, "never", accum, a)
    run_distributed(_reshard_fn, 2, "always", accum, b)
    ra, rb = torch.load(a), torch.load(b)
    assert torch.equal(ra["losses"], rb["losses"]), (ra["losses"], rb["losses"])
    assert torch.equal(ra["master"], rb["master"])


def test_per_op_selective_checkpoint_keeps_every_second_gemm():
    """``selective_ac_option = op_half_mm``: blocks are recomputed in backward except the GEMM outputs the save list
    keeps (1st, 3rd, ... of a block; forced shapes never): same losses and gradients as keeping everything, and the
    recompute really skips the kept GEMMs (reference policy: distributed/activation_checkpoint.py:186-287)."""
    from torchtitan_b200.parallel.activation_checkpoint import forced_recompute_shapes, half_mm_policy

    pdims = ParallelDims(world_size=1)
    mbs = [[x] for x in _batches(2)]
    cfg_a = _job()
    cfg_a.activation_checkpoint.mode = "selective"
    cfg_a.activation_checkpoint.selective_ac_option = "op"
    cfg_b = _job()
    cfg_b.activation_checkpoint.mode = "selective"
    cfg_b.activation_checkpoint.selective_ac_option = "op_half_mm"
    la, _, ea = _engine_steps(cfg_a, pdims, mbs, steps=2)
    lb, mb_, eb = _engine_steps(cfg_b, pdims, mbs, steps=2)
    assert torch.allclose(torch.tensor(la), torch.tensor(lb), atol=1e-6), (la, lb)
    for ua, ub in zip(ea.units, eb.units):
        assert torch.allclose(ua.master, ub.master, atol=1e-6)
    blk = next(iter(mb_.layers.values()))
    s = blk._last_sac_session
    # a llama block has four forward GEMMs: wqkv (rotated in place afterwards, so given up), wo (kept), w13 (run
    # again), w2 (kept)
    assert (s.saved, s.recomputed) == (2, 2), (s.saved, s.recomputed)
    assert not s.store                                     # every kept output was handed back and released
    # forced shapes are recomputed and do not take part in the count
    forced = forced_recompute_shapes(blk, ["attention.wo"])
    assert forced == {(blk.attention.wo.weight.shape[1], blk.attention.wo.weight.shape[0])}
    pol = half_mm_policy(forced)

    class S:
        mm_count = 0
    st = S()
    wo = next(iter(forced))
    assert [pol("mm", (1, 2), st), pol("mm", wo, st), pol("mm", (3, 4), st), pol("mm", (5, 6), st)] == [True, False, False, True]
    assert pol("attention", None, st)
