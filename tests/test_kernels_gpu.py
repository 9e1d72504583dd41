"""GPU: every hand-written kernel against the fp32 PyTorch statement of the same op."""

import math

import pytest
import torch

from torchtitan_b200.ops import ext, functional as OF, optim as optim_ops, reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_ext():
    assert ext.load(), "the sm_100a extension must be built in-tree before GPU tests run"


def _close(a, b, atol, rtol=0.0):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), float((a - b).abs().max())


@pytest.mark.parametrize("shape", [(257, 4096), (64, 8192), (1000, 128), (33, 256), (5, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("has_w", [True, False])
def test_rmsnorm(shape, dtype, has_w):
    torch.manual_seed(0)
    x = torch.randn(shape, device="cuda", dtype=dtype)
    w = (torch.randn(shape[1], device="cuda", dtype=dtype) * 0.1 + 1) if has_w else None
    dy = torch.randn(shape, device="cuda", dtype=dtype)
    y, rstd = torch.ops.tb200.rmsnorm_fwd(x, w, 1e-5)
    yr, rr = ref.rms_norm_fwd(x.float(), None if w is None else w.float(), 1e-5)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(y, yr, tol, tol)
    _close(rstd, rr, 1e-5, 1e-5)
    dx, dw = torch.ops.tb200.rmsnorm_bwd(dy, x, w, rstd)
    dxr, dwr = ref.rms_norm_bwd(dy.float(), x.float(), None if w is None else w.float(), rr)
    _close(dx, dxr, tol, tol)
    if has_w:
        _close(dw, dwr, 1e-2 * math.sqrt(shape[0]) if dtype == torch.bfloat16 else 1e-3, 1e-3)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_inplace_strided(interleaved, dtype):
    torch.manual_seed(1)
    T, Hq, Hkv, D = 300, 8, 2, 128
    table = ref.rope_table(D, 512, 500000.0, "llama").cuda()
    pos = torch.randint(0, 512, (T,), device="cuda")
    qkv = torch.randn(T, Hq + 2 * Hkv, D, device="cuda", dtype=dtype)
    orig = qkv.clone()
    view = qkv[:, :Hq + Hkv]
    torch.ops.tb200.rope_(view, table, pos, interleaved, False)
    exp = ref.rope_apply(orig[:, :Hq + Hkv].float(), table, pos, interleaved)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(qkv[:, :Hq + Hkv], exp, tol, tol)
    assert torch.equal(qkv[:, Hq + Hkv:], orig[:, Hq + Hkv:])
    torch.ops.tb200.rope_(view, table, pos, interleaved, True)
    _close(qkv, orig, 4e-2 if dtype == torch.bfloat16 else 1e-5)
    assert torch.ops.tb200.status(True) == 0


def test_rope_out_of_range_position_sets_status_without_trapping():
    table = ref.rope_table(64, 16, 10000.0).cuda()
    x = torch.randn(4, 2, 64, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([0, 3, 99, 5], device="cuda")
    torch.ops.tb200.rope_(x, table, pos, True, False)
    torch.cuda.synchronize()
    assert torch.ops.tb200.status(True) & 1
    assert torch.ops.tb200.status(False) == 0
    assert torch.isfinite(x.float()).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu(dtype):
    torch.manual_seed(2)
    gu = torch.randn(513, 2 * 1536, device="cuda", dtype=dtype)
    d = torch.randn(513, 1536, device="cuda", dtype=dtype)
    out = torch.ops.tb200.swiglu_fwd(gu)
    F = 1536
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
    _close(out, ref.swiglu_fwd(gu[:, :F].float(), gu[:, F:].float()), tol, tol)
    dgu = torch.ops.tb200.swiglu_bwd(gu, d)
    dg, du = ref.swiglu_bwd(gu[:, :F].float(), gu[:, F:].float(), d.float())
    _close(dgu[:, :F], dg, tol, tol)
    _close(dgu[:, F:], du, tol, tol)


@pytest.mark.parametrize("V,dtype", [(128256, torch.bfloat16), (2048, torch.bfloat16), (1003, torch.bfloat16),
                                     (777, torch.float32)])
def test_cross_entropy(V, dtype):
    torch.manual_seed(3)
    T = 96
    logits = (torch.randn(T, V, device="cuda") * 3).to(dtype)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    scale = torch.tensor([0.37], device="cuda")
    loss_r, dl_r, _ = ref.cross_entropy_fwd_bwd(logits.float(), labels, 0.37)
    work = logits.clone()
    row = torch.ops.tb200.cross_entropy_(work, labels, scale)
    _close(row.sum(), loss_r, 1e-2 if dtype == torch.bfloat16 else 1e-3, 1e-4)
    _close(work, dl_r, 2e-3 if dtype == torch.bfloat16 else 1e-6, 2e-2)
    assert (work[::7] == 0).all()


@pytest.mark.parametrize("gdt,sdt,pdt", [(torch.bfloat16, torch.float32, torch.bfloat16),
                                         (torch.float32, torch.float32, torch.bfloat16),
                                         (torch.float32, torch.bfloat16, torch.bfloat16),
                                         (torch.float32, torch.float32, torch.float32)])
def test_adamw(gdt, sdt, pdt):
    torch.manual_seed(4)
    n = 100003
    master = torch.randn(n, device="cuda")
    m = (torch.randn(n, device="cuda") * 0.01).to(sdt)
    v = (torch.rand(n, device="cuda") * 0.01).to(sdt)
    g = torch.randn(n, device="cuda").to(gdt)
    lowp = torch.empty(n, device="cuda", dtype=pdt)
    rm, rmm, rv = master.clone(), m.clone(), v.clone()
    rl = torch.empty(n, device="cuda", dtype=pdt)
    scale = torch.tensor([0.5], device="cuda")
    kw = dict(lr=3e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
    optim_ops.adamw_(master, g, m, v, lowp, grad_scale=scale, **kw)
    ref.adamw_step(rm, g, rmm, rv, grad_scale=0.5, out_lowp=rl, **kw)
    _close(master, rm, 1e-5, 1e-5)
    _close(m, rmm, 1e-6 if sdt == torch.float32 else 1e-3, 1e-2 if sdt == torch.bfloat16 else 1e-5)
    _close(v, rv, 1e-6 if sdt == torch.float32 else 1e-3, 1e-2 if sdt == torch.bfloat16 else 1e-5)
    _close(lowp, rl, 1e-5 if pdt == torch.float32 else 2e-2, 1e-2)


def test_adamw_skips_on_non_finite_scale():
    n = 4096
    master = torch.randn(n, device="cuda")
    before = master.clone()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda")
    lowp = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    optim_ops.adamw_(master, g, m, v, lowp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1,
                     grad_scale=torch.tensor([float("nan")], device="cuda"))
    assert torch.equal(master, before) and (m == 0).all() and (lowp == 0).all()


def test_sumsq():
    x = torch.randn(1 << 20, device="cuda")
    acc = torch.zeros(1, device="cuda")
    optim_ops.sumsq_accumulate(x, acc)
    optim_ops.sumsq_accumulate(x.bfloat16(), acc)
    exp = x.double().pow(2).sum() + x.bfloat16().double().pow(2).sum()
    _close(acc, exp.float(), 1.0, 1e-4)


def test_fused_functions_bf16_against_fp32_autograd():
    """norm_linear + rope + attention + swiglu_linear through the CUDA path vs fp32 autograd."""
    torch.manual_seed(5)
    T, D, F = 256, 512, 1024
    x = torch.randn(T, D, device="cuda")
    nw = torch.rand(D, device="cuda") + 0.5
    W13 = torch.randn(2 * F, D, device="cuda") * 0.05
    W2 = torch.randn(D, F, device="cuda") * 0.05
    g = torch.randn(T, D, device="cuda")

    def run(dtype, fused):
        xs = [t.detach().to(dtype).requires_grad_() for t in (x, nw, W13, W2)]
        if fused:
            gu = OF.norm_linear(xs[0], xs[1], xs[2], 1e-5)
            out = OF.swiglu_linear(gu, xs[3])
        else:
            xf = xs[0]
            xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * xs[1]
            gu = xn @ xs[2].t()
            out = (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ xs[3].t()
        out.backward(g.to(dtype))
        return out, [t.grad for t in xs]

    o1, g1 = run(torch.bfloat16, True)
    o2, g2 = run(torch.float32, False)
    _close(o1, o2, 5e-2, 5e-2)
    for a, b in zip(g1, g2):
        _close(a, b, 0.15 * float(b.abs().max()), 5e-2)


def test_linear_cross_entropy_cuda():
    torch.manual_seed(6)
    T, D, V = 512, 256, 4096
    h = (torch.randn(T, D, device="cuda") * 0.5)
    W = torch.randn(V, D, device="cuda") * 0.05
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[:17] = -100
    inv = torch.tensor(1.0 / (T - 17), device="cuda")
    hb, Wb = h.bfloat16().requires_grad_(), W.bfloat16().requires_grad_()
    loss = OF.linear_cross_entropy(hb, Wb, labels, inv, 4)
    loss.backward()
    hf, Wf = h.bfloat16().float().requires_grad_(), W.bfloat16().float().requires_grad_()
    l2 = torch.nn.functional.cross_entropy(hf @ Wf.t(), labels, ignore_index=-100, reduction="sum") * inv
    l2.backward()
    _close(loss, l2, 2e-2)
    _close(hb.grad, hf.grad, 0.05 * float(hf.grad.abs().max()), 5e-2)
    _close(Wb.grad, Wf.grad, 0.05 * float(Wf.grad.abs().max()), 5e-2)


def test_cuda_graph_step_matches_eager(tmp_path):
    """Forward + backward captured in a CUDA graph gives the same losses as the eager loop."""
    from torchtitan_b200.config import ConfigManager

    def run(graphs: bool):
        args = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "5",
                "--training.num_tokens_per_microbatch_per_dp_rank", "512", "--training.max_context_length", "256",
                "--debug.seed", "0", "--dump_folder", str(tmp_path / ("g" if graphs else "e")),
                "--debug.no-enable_structured_logging", "--checkpoint.no-enable", "--metrics.log_freq", "1"]
        if graphs:
            args += ["--training.no-disable_cuda_graphs"]
        tr = ConfigManager().parse_args(args).build()
        losses = []
        it = tr.batch_generator(tr.dataloader)
        for _ in range(5):
            tr.step += 1
            tr.train_step(it)
            losses.append(float(tr._last_loss))
        if graphs:
            assert tr._graph_runner is not None and len(tr._graph_runner._graphs) == 1
        tr.close()
        return losses

    eager, graph = run(False), run(True)
    assert all(abs(a - b) < 2e-2 for a, b in zip(eager, graph)), (eager, graph)
    assert graph[-1] < graph[0]


def test_per_op_checkpoint_keeps_flash_outputs_on_gpu(tmp_path):
    """``selective_ac_option = op_half_mm`` on the kernels: blocks are recomputed in backward, the flash-attention
    output and every second GEMM output are handed back from the first forward; same losses as keeping everything,
    and the attention kernel is not launched again in backward."""
    from torchtitan_b200.config import ConfigManager

    def run(opt: str):
        args = ["--module", "llama3", "--config", "llama3_debugmodel_hd128", "--training.steps", "4",
                "--training.num_tokens_per_microbatch_per_dp_rank", "512", "--training.max_context_length", "256",
                "--debug.seed", "0", "--dump_folder", str(tmp_path / opt), "--debug.no-enable_structured_logging",
                "--checkpoint.no-enable", "--metrics.log_freq", "1", "--activation_checkpoint.selective_ac_option", opt]
        tr = ConfigManager().parse_args(args).build()
        losses = []
        it = tr.batch_generator(tr.dataloader)
        for _ in range(4):
            tr.step += 1
            tr.train_step(it)
            losses.append(float(tr._last_loss))
        sess = getattr(next(iter(tr.model.layers.values())), "_last_sac_session", None)
        tr.close()
        return losses, sess

    (keep_all, _), (half, sess) = run("op"), run("op_half_mm")
    assert all(abs(a - b) < 2e-2 for a, b in zip(keep_all, half)), (keep_all, half)
    # per block: attention + two of the four GEMMs kept (wqkv is rotated in place and given up), two GEMMs recomputed
    assert sess is not None and (sess.saved, sess.recomputed) == (3, 2) and not sess.store


def test_optimizer_state_offload_matches_resident_state():
    """Pinned-host optimizer state streamed through the GPU gives the same parameters as resident
    state (up to the run-to-run last-bit differences of the atomically summed gradient norm)."""
    from tests.test_engine import T, _batches, _small_model_cfg
    from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_
    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.trainer import Trainer

    dev = torch.device("cuda", 0)
    results = []
    for offload in (False, True):
        cfg = Trainer.Config()
        cfg.training.num_tokens_per_microbatch_per_dp_rank = T
        cfg.training.max_context_length = T
        cfg.training.enable_cpu_offload = offload
        pdims = ParallelDims(world_size=1)
        with torch.device("meta"):
            model = _small_model_cfg(2).build()
        eng = parallelize_decoder(model, pdims=pdims, job_config=cfg, device=dev, seed=3)
        assert eng.offload_optimizer == offload
        opt = OptimizersContainer(OptimizersContainer.Config(lr=1e-2), engines=[eng])
        pos = torch.arange(T, device=dev)
        for tok, lab in _batches(3):
            opt.zero_grad()
            h = model(tok.to(dev), pos, return_hidden=True)
            OF.linear_cross_entropy(h, model.lm_head.weight, lab.to(dev), torch.tensor(1.0 / T, device=dev), 2).backward()
            eng.finish_backward()
            clip_grad_norm_([eng], 1.0, pdims, optimizers=opt)
            opt.step()
        if offload:
            assert all(not u.master.is_cuda and u.master.is_pinned() and not u.exp_avg.is_cuda for u in eng.units)
        results.append(torch.cat([u.flat_param[:u.numel].float() for u in eng.units]).cpu())
    d = (results[0] - results[1]).abs()
    assert float(d.max()) <= 5e-2 and float(d.mean()) <= 1e-4, (float(d.max()), float(d.mean()))
    assert float((results[0] - results[0].mean()).abs().mean()) > 1e-3


def test_activation_offload_on_gpu_matches_resident():
    from torchtitan_b200.parallel.activation_offload import OffloadStats, offload_activations

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    lin1, lin2 = torch.nn.Linear(512, 2048).to(dev), torch.nn.Linear(2048, 64).to(dev)
    x = torch.randn(4096, 512, device=dev)
    import contextlib

    def run(ctx):
        for p in list(lin1.parameters()) + list(lin2.parameters()):
            p.grad = None
        with ctx:
            y = lin2(torch.nn.functional.gelu(lin1(x))).square().sum()
        y.backward()
        torch.cuda.synchronize()
        return [p.grad.clone() for p in list(lin1.parameters()) + list(lin2.parameters())]

    ref_grads = run(contextlib.nullcontext())
    stats = OffloadStats()
    got = run(offload_activations(min_bytes=1 << 20, stats=stats))
    assert stats.tensors >= 2
    for a, b in zip(ref_grads, got):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)


def test_gemm_and_norm_are_batch_invariant():
    """A row's result does not depend on how many other rows are in the batch (no split-K, fixed tile walk)."""
    from torchtitan_b200.experiments.rl.batch_invariance import batch_invariant
    from torchtitan_b200.ops import functional as OF

    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(4096, 1024, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2048, 1024, device="cuda", generator=g) * 0.05).bfloat16()
    nw = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    with batch_invariant():
        big = OF.gemm_nt(x, w)
        for rows in (128, 256, 1000 // 8 * 8):
            small = OF.gemm_nt(x[:rows].contiguous(), w)
            assert torch.equal(big[:rows], small), rows
        nb = OF.rms_norm(x, nw, 1e-5)
        ns = OF.rms_norm(x[:8].contiguous(), nw, 1e-5)
        assert torch.equal(nb[:8], ns)
        with pytest.raises(RuntimeError, match="batch-invariant"):
            OF.gemm_nt(torch.randn(64, 36, device="cuda").bfloat16(), torch.randn(16, 36, device="cuda").bfloat16())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,C,W,docs", [(300, 256, 4, True), (64, 64, 4, False), (1000, 136, 2, True), (5, 8, 3, True)])
def test_causal_conv_silu_kernel(T, C, W, docs, dtype):
    """The fused depthwise causal convolution + SiLU (forward, dx, dw) against the tap-by-tap PyTorch form in fp32,
    with taps cut at document starts and row blocks that do not divide the sequence."""
    from torchtitan_b200.models.qwen3_5 import gdn

    g = torch.Generator(device="cuda").manual_seed(T + C)
    x32 = torch.randn(T, C, device="cuda", generator=g)
    w32 = torch.randn(C, W, device="cuda", generator=g) * 0.5
    dy32 = torch.randn(T, C, device="cuda", generator=g)
    pos = None
    if docs:
        starts = sorted({0, T // 3, T // 3 + 1, (2 * T) // 3})
        idx = torch.arange(T, device="cuda")
        st = torch.tensor(starts, device="cuda")
        pos = idx - st[torch.searchsorted(st, idx, right=True) - 1]
    x, w, dy = (t.to(dtype) for t in (x32, w32, dy32))
    xr, wr = x.float().clone().requires_grad_(), w.float().clone().requires_grad_()
    orig = gdn._conv_kernel_ok
    gdn._conv_kernel_ok = lambda *_: False
    try:
        ref = gdn.causal_conv_silu(xr, wr, pos)
        ref.backward(dy.float())
    finally:
        gdn._conv_kernel_ok = orig
    xk, wk = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    assert gdn._conv_kernel_ok(xk, wk)
    out = gdn.causal_conv_silu(xk, wk, pos)
    out.backward(dy)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for got, want in ((out, ref), (xk.grad, xr.grad), (wk.grad, wr.grad)):
        err = (got.float() - want).abs().max().item()
        assert err <= tol * (want.abs().max().item() + 1.0), (err, want.abs().max().item())


def test_mla_assemble_kernel_matches_separate_ops():
    """The fused multi-head-latent-attention assembly (rotary q_pe / k_pe, [nope | pe] queries and keys, contiguous
    values) and its backward against the separate rotary / concatenate / expand operators in fp32."""
    from torchtitan_b200.models.common.mla import _MLAAssembleFn

    T, H, dn, dr, dv, rank = 200, 4, 32, 16, 32, 64
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn(T, H, dn + dr, device="cuda", generator=g).bfloat16()
    kv = torch.randn(T, H, dn + dv, device="cuda", generator=g).bfloat16()
    kv_a = torch.randn(T, rank + dr, device="cuda", generator=g).bfloat16()
    table = ref.rope_table(dr, 512, 10000.0).cuda()
    pos = torch.randint(0, 512, (T,), device="cuda")
    grads = [torch.randn(T, H, dn + dr, device="cuda", generator=g).bfloat16(),
             torch.randn(T, H, dn + dr, device="cuda", generator=g).bfloat16(),
             torch.randn(T, H, dv, device="cuda", generator=g).bfloat16()]

    def separate(q, kv, kv_a):
        q_pe = ref.rope_apply(q[:, :, dn:], table, pos, True)
        k_pe = ref.rope_apply(kv_a[:, rank:].reshape(T, 1, dr), table, pos, True)
        return (torch.cat([q[:, :, :dn], q_pe], -1), torch.cat([kv[:, :, :dn], k_pe.expand(T, H, dr)], -1), kv[:, :, dn:])

    a = [t.float().requires_grad_() for t in (q, kv, kv_a)]
    want = separate(*a)
    torch.autograd.backward(want, [x.float() for x in grads])
    b = [t.clone().requires_grad_() for t in (q, kv, kv_a)]
    got = _MLAAssembleFn.apply(b[0], b[1], b[2][:, rank:], table, pos, dn, dr, dv)
    torch.autograd.backward(got, grads)
    assert got[2].is_contiguous()
    for x, y in zip(got, want):
        assert (x.float() - y).abs().max().item() <= 2e-2 * y.abs().max().item() + 1e-3
    for x, y in zip(b, a):
        assert (x.grad.float() - y.grad).abs().max().item() <= 2e-2 * y.grad.abs().max().item() + 2e-2
    assert (b[2].grad[:, :rank] == 0).all()
    assert OF.settings is not None and torch.ops.tb200.status(True) == 0
