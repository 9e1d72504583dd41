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
