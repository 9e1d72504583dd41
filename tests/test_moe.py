"""MoE layer: routing math, grouped experts vs a per-token loop, expert parallel vs local."""

import torch

from tests.dist_utils import run_distributed
from torchtitan_b200.models.common.moe import GroupedExperts, MoE, RoutedExperts, TokenChoiceTopKRouter


def _moe(E=8, K=2, dim=16, hidden=24, shared=0):
    cfg = MoE.Config(dim=dim, hidden_dim=hidden, num_experts=E, top_k=K, shared_hidden_dim=shared,
                     router=TokenChoiceTopKRouter.Config(score_func="softmax", route_norm=True))
    m = cfg.build()
    m.init_states(seed=1)
    return m


def _loop_reference(m, x):
    top, sel, _ = m.router(x, m.expert_bias_E)
    ex = m.routed_experts.inner_experts
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(sel.shape[1]):
            e = int(sel[t, k])
            h = torch.nn.functional.silu(x[t] @ ex.w1_EFD[e].t()) * (x[t] @ ex.w3_EFD[e].t())
            out[t] += top[t, k] * (h @ ex.w2_EDF[e].t())
    return out


def test_moe_matches_per_token_loop():
    torch.manual_seed(0)
    m = _moe()
    x = torch.randn(12, 16)
    y = m(x)
    assert torch.allclose(y, _loop_reference(m, x), atol=1e-5)
    assert m.tokens_per_expert_E.sum() == 24
    y.sum().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_shared_experts_and_bias_only_affects_selection():
    torch.manual_seed(1)
    m = _moe(shared=32)
    x = torch.randn(6, 16)
    y0 = m(x)
    m.expert_bias_E += 100.0  # uniform shift: same selection, gate values unchanged
    assert torch.allclose(m(x), y0, atol=1e-6)


def _ep_fn(rank, world, out_path):
    import torch.distributed as dist

    from torchtitan_b200.parallel.expert_parallel import EPContext

    torch.manual_seed(0)
    full = _moe(E=8, K=2)
    x_all = torch.randn(2, 10, 16)
    ref_out = [full(x_all[r]) for r in range(world)]
    # expert-parallel copy holding experts [4r, 4r+4)
    local = _moe(E=8, K=2)
    ie = local.routed_experts.inner_experts
    n = 8 // world
    for name in ("w1_EFD", "w2_EDF", "w3_EFD"):
        setattr(ie, name, torch.nn.Parameter(getattr(ie, name).detach()[rank * n:(rank + 1) * n].clone()))
    ie.num_experts = n
    local.routed_experts.ep = EPContext(group=dist.group.WORLD, size=world, rank=rank)
    x = x_all[rank].clone().requires_grad_()
    y = local(x)
    ok = torch.allclose(y, ref_out[rank], atol=1e-5)
    y.sum().backward()
    xr = x_all[rank].clone().requires_grad_()
    full.zero_grad()
    # gradient wrt x on this rank only depends on this rank's tokens
    full(xr).sum().backward()
    ok = ok and torch.allclose(x.grad, xr.grad, atol=1e-5)
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save(flag, out_path)


def test_expert_parallel_matches_local(tmp_path):
    out = str(tmp_path / "ep.pt")
    run_distributed(_ep_fn, 2, out)
    assert float(torch.load(out)) == 1.0


def test_force_load_balance_flag_reaches_every_router(tmp_path):
    """``debug.moe_force_load_balance`` assigns experts round-robin in every mixture-of-experts layer (balanced counts)."""
    from torchtitan_b200.config import ConfigManager

    cfg = ConfigManager().parse_args([
        "--module", "qwen3", "--config", "qwen3_moe_tiny", "--debug.moe_force_load_balance",
        "--training.num_tokens_per_microbatch_per_dp_rank", "64", "--training.max_context_length", "64",
        "--debug.no-enable_structured_logging", "--dump_folder", str(tmp_path)])
    t = cfg.build()
    routers = [blk.moe.router for blk in t.model.layers.values() if blk.moe is not None]
    assert routers and all(r.config._debug_force_load_balance for r in routers)
    _, sel, counts = routers[0](torch.randn(64, 64), None)
    assert torch.equal(counts, torch.full((8,), 16.0)) and sel.shape == (64, 2)
    t.close()
