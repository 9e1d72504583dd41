"""GPU: the native MoE path (fused router, padded permute, grouped tcgen05 GEMMs, combine) against
the same layer evaluated in fp32 on the CPU."""

import copy

import pytest
import torch

from torchtitan_b200.models.common.moe import MoE, TokenChoiceTopKRouter
from torchtitan_b200.ops import ext

pytestmark = pytest.mark.gpu


def _build(score_func, route_norm, E=8, K=2, dim=256, hidden=384, shared=0):
    cfg = MoE.Config(dim=dim, hidden_dim=hidden, num_experts=E, top_k=K, shared_hidden_dim=shared,
                     router=TokenChoiceTopKRouter.Config(score_func=score_func, route_norm=route_norm, route_scale=1.5))
    m = cfg.build()
    m.init_states(seed=3)
    return m


@pytest.mark.parametrize("score_func,route_norm", [("softmax", True), ("sigmoid", False)])
def test_native_moe_matches_cpu_reference(score_func, route_norm):
    ext.require()
    torch.manual_seed(0)
    ref = _build(score_func, route_norm)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())  # both sides start from bf16-representable weights
    gpu = copy.deepcopy(ref).cuda().bfloat16()
    gpu.expert_bias_E = gpu.expert_bias_E.float()
    gpu.tokens_per_expert_E = gpu.tokens_per_expert_E.float()
    assert gpu.routed_experts.inner_experts.native_ok(torch.empty(1, 256, device="cuda", dtype=torch.bfloat16))
    x = (torch.randn(300, 256) * 0.5).bfloat16().float()
    xg = x.cuda().bfloat16().requires_grad_()
    xr = x.clone().requires_grad_()
    yg = gpu(xg)
    yr = ref(xr)
    assert torch.equal(gpu.tokens_per_expert_E.cpu(), ref.tokens_per_expert_E)
    assert (yg.float().cpu() - yr).abs().max().item() <= 3e-2 * yr.abs().max().item() + 1e-3
    g = torch.randn_like(yr)
    yg.backward(g.cuda().bfloat16())
    yr.backward(g.bfloat16().float())
    torch.cuda.synchronize()
    assert torch.ops.tb200.gemm_status(True) == 0
    assert (xg.grad.float().cpu() - xr.grad).abs().max().item() <= 4e-2 * xr.grad.abs().max().item() + 1e-3
    for (n, pg), (_, pr) in zip(gpu.named_parameters(), ref.named_parameters()):
        err = (pg.grad.float().cpu() - pr.grad).abs().max().item()
        assert err <= 5e-2 * pr.grad.abs().max().item() + 2e-3, (n, err)


def test_router_kernel_matches_reference_selection():
    from torchtitan_b200.ops import moe_ops, reference as ref

    ext.require()
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(1000, 128, device="cuda", generator=g)
    bias = torch.randn(128, device="cuda", generator=g) * 0.1
    for func, norm in (("softmax", True), ("sigmoid", True), ("sigmoid", False)):
        top, sel, counts = moe_ops.router_topk(logits, bias, 8, func, norm, 2.5)
        rtop, rsel, rcounts = ref.router_topk(logits, 8, func, bias, norm, 2.5)
        assert torch.equal(sel.long().sort(dim=-1).values, rsel.sort(dim=-1).values)
        assert torch.equal(counts, rcounts)
        assert torch.allclose(top.sort(dim=-1).values, rtop.sort(dim=-1).values, atol=1e-5, rtol=1e-4)


def _layout_reference(selected, all_counts, me, align=128):
    """The expert-parallel layout in plain tensor ops: rows of an expert start at a multiple of ``align``,
    lower source ranks first, token order inside a source rank."""
    n, E = all_counts.shape
    El = E // n
    T, K = selected.shape
    tot = all_counts.sum(0)
    padded = ((tot + align - 1) // align * align).view(n, El)
    offs = torch.zeros(n, El + 1, dtype=torch.int64)
    offs[:, 1:] = torch.cumsum(padded, 1)
    base = offs[:, :-1].reshape(-1) + all_counts[:me].sum(0)
    flat = selected.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    e_sorted = flat[order]
    c = all_counts[me]
    start = torch.cumsum(c, 0) - c
    pos = torch.arange(T * K) - start[e_sorted]
    dest_row = torch.empty(T * K, dtype=torch.int64)
    dest_row[order] = base[e_sorted] + pos
    return (flat // El).view(T, K), dest_row.view(T, K), offs[me], tot.view(n, El)[me]


def test_ep_layout_kernel_matches_reference():
    """Device-side layout of two emulated ranks (the count table is filled by hand) against tensor ops."""
    ops = ext.require()
    torch.manual_seed(3)
    n, E, T, K = 2, 16, 3000, 4
    sels = [torch.stack([torch.randperm(E)[:K] for _ in range(T)]).int() for _ in range(n)]
    all_counts = torch.stack([torch.bincount(s.reshape(-1).long(), minlength=E) for s in sels])
    table = all_counts.int().cuda()
    for me in range(n):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = ops.ep_layout(sels[me].cuda(), table, me, 1 << 20, 128, status)
        want = _layout_reference(sels[me], all_counts, me)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for g, w in zip(got, want):
            assert torch.equal(g.cpu().long(), w.long())
    # a capacity that is too small: the slots that do not fit are dropped (row -1) and the status word says so
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cap = 4096
    dest_rank, dest_row, my_offs, _ = ops.ep_layout(sels[0].cuda(), table, 0, cap, 128, status)
    torch.cuda.synchronize()
    assert int(status.item()) & 8
    assert int(dest_row.max()) < cap and int((dest_row < 0).sum()) > 0 and int(my_offs[-1]) <= cap
