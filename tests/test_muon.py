"""DistMuon on the flat-sharded engine: Newton-Schulz numerics, one step against the restated math,
two ranks against one rank."""

import torch

from tests.dist_utils import run_distributed
from tests.test_engine import T, _batches, _build_engine, _job, _small_model_cfg
from torchtitan_b200.components.optimizer import OptimizersContainer, ParamGroupConfig, clip_grad_norm_
from torchtitan_b200.ops import functional as OF
from torchtitan_b200.parallel.muon import adjust_lr, newton_schulz
from torchtitan_b200.parallel.parallel_dims import ParallelDims

MUON_PATTERN = r"layers\.\d+\.(attention\.(wqkv|wo)|feed_forward\.w(13|1|2|3))\.weight$"


def _opt_config(lr=2e-2):
    return OptimizersContainer.Config(
        lr=lr,
        param_groups=[ParamGroupConfig(pattern=MUON_PATTERN, optimizer_name="DistMuon",
                                       optimizer_kwargs={"lr": lr, "adjust_lr_fn": "match_rms_adamw"})],
    )


def test_newton_schulz_orthogonalises():
    g = torch.Generator().manual_seed(0)
    for shape in [(64, 160), (192, 48)]:
        x = torch.randn(*shape, generator=g)
        d = newton_schulz(x).float()
        assert d.shape == x.shape
        sv = torch.linalg.svdvals(d)
        assert sv.max() < 1.3 and sv.min() > 0.5, (sv.min(), sv.max())
        # same singular vectors as the input: U^T D V is close to diagonal-positive
        u, _, vh = torch.linalg.svd(x, full_matrices=False)
        core = u.t() @ d @ vh.t()
        off = core - torch.diag(torch.diagonal(core))
        assert off.abs().max() < 0.08 and torch.diagonal(core).min() > 0.5


def test_adjust_lr_rules():
    assert adjust_lr(1.0, None, 8, 2) == 2.0 and adjust_lr(1.0, "original", 2, 8) == 1.0
    assert abs(adjust_lr(1.0, "match_rms_adamw", 100, 400) - 4.0) < 1e-12
    assert abs(adjust_lr(1.0, "spectral_unclamped", 2, 8) - 0.5) < 1e-12


def _steps(pdims, microbatches_per_step, accum=1, steps=2):
    cfg = _job(accum_tokens=accum * T * pdims.dp_degree if accum > 1 else -1)
    mc, model, eng = _build_engine(cfg, pdims, accum)
    opt = OptimizersContainer(_opt_config(), engines=[eng])
    assert any("wqkv" in n or "wq" in n for n in opt.group_members[0])
    pos = torch.arange(T)
    grads = None
    for s in range(steps):
        opt.zero_grad()
        mbs = microbatches_per_step[s]
        n_tok = torch.tensor(float(T * len(mbs) * pdims.dp_degree))
        for tok, lab in mbs:
            h = model(tok, pos, return_hidden=True)
            OF.linear_cross_entropy(h, model.lm_head.weight, lab, 1.0 / n_tok, 4).backward()
            eng.finish_backward()
        clip_grad_norm_([eng], 1e9, pdims, optimizers=opt)
        opt.step()
    return model, eng, opt


def test_one_step_matches_restated_math():
    pdims = ParallelDims(world_size=1)
    b = _batches(1)
    model, eng, opt = _steps(pdims, [[b[0]]], steps=1)
    # the same step by hand on a plain copy of the model
    mc = _small_model_cfg()
    plain = mc.build()
    plain.init_states(seed=7)
    tok, lab = b[0]
    logits = plain(tok, torch.arange(T))
    (torch.nn.functional.cross_entropy(logits.float(), lab, reduction="sum") / T).backward()
    import re

    lr, wd, beta = 2e-2, 0.1, 0.95
    checked = 0
    for (n, p), (n2, q) in zip(plain.named_parameters(), model.named_parameters()):
        assert n == n2
        if not re.search(MUON_PATTERN, n):
            continue
        g = p.grad.float()
        m = g * (1 - beta)                        # lerp(0, g, 1 - beta)
        prepared = torch.lerp(g, m, beta)         # Nesterov blend
        d = newton_schulz(prepared.bfloat16()).float()
        want = p.detach() * (1 - lr * wd) - adjust_lr(lr, "match_rms_adamw", *p.shape) * d
        # the direction is rounded to bf16 on its way through the reduce-scatter buffer
        assert torch.allclose(q.detach(), want, atol=2e-2 * lr * 0.2 * max(p.shape) ** 0.5 + 1e-6), (n, (q - want).abs().max())
        assert (q.detach() - p.detach()).abs().max() > 1e-4
        checked += 1
    assert checked >= 4


def _rank_fn(rank, world, out_path):
    pdims = ParallelDims(world_size=world, rank=rank).build()
    b = _batches(4)
    model, eng, opt = _steps(pdims, [[b[2 * s + rank]] for s in range(2)])
    if rank == 0:
        torch.save({n: p.detach().clone() for n, p in model.named_parameters()}, out_path)


def test_two_ranks_match_one_rank(tmp_path):
    out = str(tmp_path / "muon2.pt")
    run_distributed(_rank_fn, 2, out)
    got = torch.load(out)
    pdims = ParallelDims(world_size=1)
    b = _batches(4)
    model, _, _ = _steps(pdims, [b[0:2], b[2:4]], accum=2)
    import re

    for n, p in model.named_parameters():
        if re.search(MUON_PATTERN, n):
            # bf16 Newton-Schulz amplifies last-bit input differences along weak singular directions
            d = (p - got[n]).abs()
            assert d.max() <= 1e-2 and d.mean() <= 3e-4, (n, d.max(), d.mean())
        else:
            # AdamW's g / (|g| + eps) turns last-bit differences of near-zero gradients into up to one lr
            d = (p - got[n]).abs()
            assert d.max() <= 3e-2 and d.mean() <= 2e-4, (n, d.max(), d.mean())
