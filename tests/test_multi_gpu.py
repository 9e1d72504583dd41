"""Multi-GPU (>= 2 devices): NVLink in-kernel collectives against the NCCL path, and the bounded wait."""

import pytest
import torch

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def test_bounded_wait_reports_timeout_without_trapping():
    """A barrier whose peer never arrives must set the status word and return (single GPU:
    both 'ranks' point at local flag arrays and nothing ever sets the peer's slot)."""
    from torchtitan_b200.ops import ext

    assert ext.load()
    a = torch.zeros(64, dtype=torch.int32, device="cuda")
    b = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.ops.tb200.symm_barrier([a.data_ptr(), b.data_ptr()], 0, epoch, status, 2_000_000, None)  # ~1 ms of cycles
    torch.cuda.synchronize()
    assert int(status.item()) & 4
    assert int(epoch.item()) == 1  # the kernel advanced the device-side epoch
    assert int(b[0].item()) == 1  # our own arrival was published to the "peer"
    # the context is still healthy
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def _train(rank, world, comm, out_path, reshard="never"):
    import torch.distributed as dist

    from tests.test_engine import T, _batches, _small_model_cfg
    from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_
    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.trainer import Trainer

    dev = torch.device("cuda", rank)
    cfg = Trainer.Config()
    cfg.training.num_tokens_per_microbatch_per_dp_rank = T
    cfg.training.max_context_length = T
    cfg.parallelism.fsdp_comm = comm
    cfg.parallelism.fsdp_reshard_after_forward = reshard
    pdims = ParallelDims(world_size=world, rank=rank).build()
    mc = _small_model_cfg(3)
    with torch.device("meta"):
        model = mc.build()
    eng = parallelize_decoder(model, pdims=pdims, job_config=cfg, device=dev, seed=3)
    opt = OptimizersContainer(OptimizersContainer.Config(lr=1e-2), engines=[eng])
    b = _batches(8)
    pos = torch.arange(T, device=dev)
    losses = []
    for s in range(4):
        tok, lab = (t.to(dev) for t in b[2 * s + rank % 2])
        opt.zero_grad()
        h = model(tok, pos, return_hidden=True)
        loss = OF.linear_cross_entropy(h, model.lm_head.weight, lab, torch.tensor(1.0 / (T * world), device=dev), 2)
        loss.backward()
        eng.finish_backward()
        clip_grad_norm_([eng], 1.0, pdims, optimizers=opt)
        opt.step()
        losses.append(loss.detach())
    eng.check_status()
    t = torch.stack(losses)
    dist.all_reduce(t)
    assert eng.sharded_params == (reshard == "always")
    full = torch.cat([u.master for u in eng.units])    # this rank's fp32 shards
    if rank == 0:
        torch.save({"losses": t.cpu(), "params": full.cpu()}, out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_nvlink_engine_matches_nccl(tmp_path):
    a, b = str(tmp_path / "nccl.pt"), str(tmp_path / "nvl.pt")
    run_distributed(_train, 2, "nccl", a, backend="nccl")
    run_distributed(_train, 2, "nvlink", b, backend="nccl")
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra["losses"], rb["losses"], atol=2e-2), (ra["losses"], rb["losses"])
    # race detection: with the gradient buffers poisoned (NaN) as soon as every rank has finished reading them, a
    # stale read anywhere in the step would turn the losses into NaN; they must stay what they were
    c = str(tmp_path / "canary.pt")
    run_distributed(_train, 2, "nvlink", c, backend="nccl", env={"TB200_SYMM_CANARY": "1"})
    rc = torch.load(c)
    assert torch.isfinite(rc["losses"]).all() and torch.allclose(rb["losses"], rc["losses"], atol=1e-3), rc["losses"]
    # AdamW's g / (|g| + eps) turns last-bit differences of near-zero gradients (reduction order) into
    # up to one learning rate per step for single elements: bound the maximum loosely, the mean tightly
    d = (ra["params"] - rb["params"]).abs()
    assert float(d.max()) <= 0.1 and float(d.mean()) <= 1e-3, (float(d.max()), float(d.mean()))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm", ["nccl", "nvlink"])
def test_sharded_parameters_match_resident(tmp_path, comm):
    """fsdp_reshard_after_forward = always (per-unit gathers into rotating slots, prefetch on the communication
    stream) against the resident layout, over NCCL and over the peer-load kernels."""
    a, b = str(tmp_path / "never.pt"), str(tmp_path / "always.pt")
    run_distributed(_train, 2, comm, a, "never", backend="nccl")
    run_distributed(_train, 2, comm, b, "always", backend="nccl")
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra["losses"], rb["losses"], atol=1e-3), (ra["losses"], rb["losses"])
    # AdamW's g / (|g| + eps) turns last-bit differences of near-zero gradients into up to one learning rate per
    # step for single elements (the two layouts update through different kernels): loose maximum, tight mean
    d = (ra["params"] - rb["params"]).abs()
    assert float(d.max()) <= 0.1 and float(d.mean()) <= 1e-3, (float(d.max()), float(d.mean()))


def _rs_ag(rank, world, out_path):
    """reduce_scatter_pull and the fused AdamW+all-gather against torch math on raw buffers."""
    import torch.distributed as dist

    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.symm import SymmetricArena

    dev = torch.device("cuda", rank)
    pdims = ParallelDims(world_size=world, rank=rank).build()
    g = pdims.group("fsdp")
    n = 1 << 20
    arena = SymmetricArena(pdims, dev)
    arena.reserve(g, 2 * n * 2)
    grad = arena.alloc(n, torch.bfloat16, g)
    torch.manual_seed(100 + rank)
    grad.copy_(torch.randn(n, device=dev))
    shard = torch.zeros(n // world, dtype=torch.float32, device=dev)
    if rank == 1:
        torch.cuda._sleep(400_000_000)     # arrival skew: this rank reaches the collective ~0.2 s late
    arena.reduce_scatter_accumulate(grad, shard, g, accumulate=False)
    gathered = [torch.empty(n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    dist.all_gather(gathered, grad)
    exp = sum(t.float() for t in gathered)[rank * (n // world):(rank + 1) * (n // world)]
    ok1 = torch.allclose(shard, exp, atol=1e-5)
    if rank == 0:
        torch.cuda._sleep(400_000_000)     # and the other rank late for the second one
    arena.reduce_scatter_accumulate(grad, shard, g, accumulate=True)
    ok2 = torch.allclose(shard, 2 * exp, atol=1e-4)
    for a in arena._arenas.values():
        assert int(a.status.item()) == 0
    if rank == 0:
        torch.save({"ok1": ok1, "ok2": ok2}, out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_reduce_scatter_pull(tmp_path):
    out = str(tmp_path / "rs.pt")
    run_distributed(_rs_ag, 2, out, backend="nccl")
    r = torch.load(out)
    assert r["ok1"] and r["ok2"]


def _adamw_ag(rank, world, out_path):
    """The fused AdamW + all-gather kernel on raw buffers; with TB200_MULTICAST=1 in the environment
    the refreshed weights travel as multimem stores through the switch, else as per-peer stores."""
    import torch.distributed as dist

    from torchtitan_b200.parallel.fsdp import FlatUnit
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.symm import SymmetricArena

    dev = torch.device("cuda", rank)
    pdims = ParallelDims(world_size=world, rank=rank).build()
    g = pdims.group("fsdp")
    n = 1 << 18
    arena = SymmetricArena(pdims, dev)
    arena.reserve(g, 2 * n * 2)
    unit = FlatUnit("u", [], g, world, rank)
    unit.padded, unit.shard_numel = n, n // world
    unit.flat_param = arena.alloc(n, torch.bfloat16, g)
    unit.flat_param.zero_()
    S = n // world
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    unit.master = torch.randn(S, device=dev, generator=gen)
    unit.exp_avg = torch.zeros(S, device=dev)
    unit.exp_avg_sq = torch.zeros(S, device=dev)
    grad = torch.randn(S, device=dev, generator=gen)
    ref_master = unit.master.clone()
    groups = [dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)]
    arena.barrier_all()
    arena.adamw_allgather(unit, [(0, 0, S)], groups, 1, torch.ones(1, device=dev), grad)
    arena.barrier_all()
    torch.cuda.synchronize()
    # reference: AdamW step 1 on the shard, then all-gather of the bf16 weights
    m = 0.1 * grad
    v = 0.05 * grad * grad
    upd = (m / (1 - 0.9)) / ((v / (1 - 0.95)).sqrt() + 1e-8)
    exp_shard = (ref_master * (1 - 1e-2 * 0.1) - 1e-2 * upd).bfloat16()
    want = torch.empty(n, dtype=torch.bfloat16, device=dev)
    dist.all_gather_into_tensor(want, exp_shard)
    err = (unit.flat_param.float() - want.float()).abs().max()
    used_mc = 1.0 if next(iter(arena._arenas.values())).mc_base else 0.0
    st = float(next(iter(arena._arenas.values())).status.item())
    t = torch.stack([err, torch.tensor(st, device=dev), torch.tensor(used_mc, device=dev)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        torch.save(t.cpu(), out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_adamw_allgather_multicast_matches_peer_stores(tmp_path):
    """The only test that binds memory to an NVSwitch multicast object: multimem.st against per-peer stores."""
    a, b = str(tmp_path / "peer.pt"), str(tmp_path / "mc.pt")
    run_distributed(_adamw_ag, 2, a, backend="nccl")
    run_distributed(_adamw_ag, 2, b, backend="nccl", env={"TB200_MULTICAST": "1", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "0"})
    ra, rb = torch.load(a), torch.load(b)
    assert ra[1] == 0 and rb[1] == 0, "a bounded wait expired"
    assert ra[2] == 0, "the default test environment must not use multicast"
    assert ra[0] <= 1e-2 and rb[0] <= 1e-2, (ra, rb)


def _fused_tp(rank, world, out_path):
    """All-gather -> GEMM and GEMM -> reduce-scatter kernels against NCCL + fp32 matmul."""
    import torch.distributed as dist

    from torchtitan_b200.parallel.tp_fused import FusedTP, all_gather_linear, linear_reduce_scatter

    dev = torch.device("cuda", rank)
    ftp = FusedTP(dist.group.WORLD, dev, nbytes=256 << 20)
    T, K, N = 1024 * world, 512, 768
    S = T // world
    res = {}
    for it in range(3):   # three rounds: both buffers of each pair get reused
        g = torch.Generator(device=dev).manual_seed(10 * it + rank)
        x = (torch.randn(S, K, device=dev, generator=g) * 0.5).bfloat16().requires_grad_()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16().requires_grad_()
        y = all_gather_linear(x, w, ftp)
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x.detach())
        x_full = torch.cat(xs).float()
        ref = x_full @ w.detach().float().t()
        e1 = (y.float() - ref).abs().max().item() / ref.abs().max().item()
        dy = (torch.randn(T, N, device=dev, generator=g) * 0.1).bfloat16()
        y.backward(dy)
        dxp = dy.float() @ w.detach().float()          # partial: summed over ranks, my rows
        dist.all_reduce(dxp)
        e2 = (x.grad.float() - dxp[rank * S:(rank + 1) * S]).abs().max().item() / dxp.abs().max().item()
        e3 = (w.grad.float() - dy.float().t() @ x_full).abs().max().item() / (dy.float().t() @ x_full).abs().max().item()
        # row-parallel
        x2 = (torch.randn(T, K, device=dev, generator=g) * 0.5).bfloat16().requires_grad_()
        w2 = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16().requires_grad_()
        y2 = linear_reduce_scatter(x2, w2, ftp)
        ref2 = x2.detach().float() @ w2.detach().float().t()
        dist.all_reduce(ref2)
        e4 = (y2.float() - ref2[rank * S:(rank + 1) * S]).abs().max().item() / ref2.abs().max().item()
        dy2 = (torch.randn(S, N, device=dev, generator=g) * 0.1).bfloat16()
        y2.backward(dy2)
        dys = [torch.empty_like(dy2) for _ in range(world)]
        dist.all_gather(dys, dy2)
        dy_full = torch.cat(dys).float()
        e5 = (x2.grad.float() - dy_full @ w2.detach().float()).abs().max().item() / (dy_full @ w2.detach().float()).abs().max().item()
        wref = dy_full.t() @ x2.detach().float()
        e6 = (w2.grad.float() - wref).abs().max().item() / wref.abs().max().item()
        res[it] = [e1, e2, e3, e4, e5, e6]
    torch.cuda.synchronize()
    status = int(ftp.arena.status.item()) | int(torch.ops.tb200.gemm_status(True))
    t = torch.tensor([max(v) for v in res.values()] + [float(status)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        torch.save({"errs": t.cpu(), "detail": res}, out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_tensor_parallel_gemms(tmp_path):
    out = str(tmp_path / "ftp.pt")
    run_distributed(_fused_tp, 2, out, backend="nccl")
    r = torch.load(out)
    assert r["errs"][-1] == 0, "a bounded wait expired"
    assert (r["errs"][:-1] < 3e-2).all(), r


def _train_tp(rank, world, tp_comm, out_path):
    import torch.distributed as dist

    from tests.test_engine import _small_model_cfg
    from torchtitan_b200.components.optimizer import OptimizersContainer, clip_grad_norm_
    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.trainer import Trainer

    Tn = 1024
    dev = torch.device("cuda", rank)
    cfg = Trainer.Config()
    cfg.training.num_tokens_per_microbatch_per_dp_rank = Tn
    cfg.training.max_context_length = Tn
    cfg.parallelism.tensor_parallel_degree = world
    cfg.parallelism.tp_comm = tp_comm
    cfg.parallelism.tp_symm_bytes = 64 << 20
    pdims = ParallelDims(world_size=world, rank=rank, tp=world).build()
    mc = _small_model_cfg(2)
    for blk in mc.layers:
        blk.attention.rope.max_context_length = Tn
    with torch.device("meta"):
        model = mc.build()
    eng = parallelize_decoder(model, pdims=pdims, job_config=cfg, device=dev, seed=3)
    if tp_comm == "nvlink":
        assert model.tp.fused is not None
    opt = OptimizersContainer(OptimizersContainer.Config(lr=1e-2), engines=[eng])
    from torchtitan_b200.components.loss import LinearCrossEntropyLoss

    loss_fn = LinearCrossEntropyLoss()
    loss_fn.set_lm_head(model.lm_head, tp=model.tp)
    g = torch.Generator().manual_seed(0)
    pos = torch.arange(Tn, device=dev)
    losses = []
    for s in range(3):
        ids = torch.randint(0, 2048, (Tn + 1,), generator=g)
        tok, lab = ids[:-1].to(dev), ids[1:].to(dev)
        opt.zero_grad()
        h = model(tok, pos, return_hidden=True)
        loss = loss_fn(h, lab, torch.tensor(float(Tn), device=dev))
        loss.backward()
        eng.finish_backward()
        clip_grad_norm_([eng], 1.0, pdims, optimizers=opt)
        opt.step()
        losses.append(loss.detach())
    eng.check_status()
    torch.cuda.synchronize()
    assert int(torch.ops.tb200.gemm_status(True)) == 0
    if rank == 0:
        torch.save({"losses": torch.stack(losses).cpu()}, out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_fused_matches_nccl(tmp_path):
    a, b = str(tmp_path / "tp_nccl.pt"), str(tmp_path / "tp_nvl.pt")
    run_distributed(_train_tp, 2, "nccl", a, backend="nccl")
    run_distributed(_train_tp, 2, "nvlink", b, backend="nccl")
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra["losses"], rb["losses"], atol=3e-2), (ra["losses"], rb["losses"])


def _ep_nvlink(rank, world, out_path):
    """Expert parallelism: NVLink scatter / gather kernels against the NCCL all-to-all dispatcher."""
    import copy

    import torch.distributed as dist

    from torchtitan_b200.models.common.moe import MoE, TokenChoiceTopKRouter
    from torchtitan_b200.parallel.ep_nvlink import EPNvlink
    from torchtitan_b200.parallel.expert_parallel import EPContext

    dev = torch.device("cuda", rank)
    E, K, dim, hidden, T = 8, 2, 256, 384, 600
    cfg = MoE.Config(dim=dim, hidden_dim=hidden, num_experts=E, top_k=K,
                     router=TokenChoiceTopKRouter.Config(score_func="softmax", route_norm=True))
    base = cfg.build()
    base.init_states(seed=5)
    n = E // world

    def make(comm):
        m = copy.deepcopy(base)
        ie = m.routed_experts.inner_experts
        for name in ("w1_EFD", "w2_EDF", "w3_EFD"):
            setattr(ie, name, torch.nn.Parameter(getattr(ie, name).detach()[rank * n:(rank + 1) * n].clone()))
        ie.num_experts = n
        m = m.to(dev).bfloat16()
        m.expert_bias_E = m.expert_bias_E.float()
        m.tokens_per_expert_E = m.tokens_per_expert_E.float()
        ep = EPContext(group=dist.group.WORLD, size=world, rank=rank, comm=comm)
        if comm == "nvlink":
            ep.nvlink = EPNvlink(dist.group.WORLD, dev, world * T * K + n * 128, dim, E)
        m.routed_experts.ep = ep
        return m

    res = []
    models = {comm: make(comm) for comm in ("nccl", "nvlink")}
    # a third model on the exact mode of the NVLink dispatcher (worst-case buffers, received row count read on the
    # host per exchange, kept rows and activations of that size)
    models["nvlink_exact"] = make("nvlink")
    models["nvlink_exact"].routed_experts.ep.nvlink.exact = True
    for it in range(2):   # two rounds: the symmetric buffers are reused
        g = torch.Generator(device=dev).manual_seed(50 + 7 * it + rank)
        x = (torch.randn(T, dim, device=dev, generator=g) * 0.5).bfloat16()
        dy = (torch.randn(T, dim, device=dev, generator=g) * 0.1).bfloat16()
        outs = {}
        for comm in ("nccl", "nvlink", "nvlink_exact"):
            m = models[comm]
            m.zero_grad()
            xi = x.clone().requires_grad_()
            y = m(xi)
            y.backward(dy)
            outs[comm] = (y.detach().float(), xi.grad.float(), m.routed_experts.inner_experts.w1_EFD.grad.float(),
                          m.router.gate.weight.grad.float())
        for other in ("nvlink", "nvlink_exact"):
            for a, b in zip(outs["nccl"], outs[other]):
                res.append((a - b).abs().max().item() / (a.abs().max().item() + 1e-6))
    # the NVLink dispatcher has no host read and no library collective: the layer's forward can be captured in a
    # CUDA graph (a synchronisation during capture would raise) and the replay reproduces the eager result
    m = models["nvlink"]
    with torch.no_grad():
        x_static = x.clone()
        y_eager = m(x_static).float()
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            m(x_static)                                  # warm-up on the capture stream
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_static = m(x_static)
        graph.replay()
        graph.replay()
        torch.cuda.synchronize()
        res.append((y_static.float() - y_eager).abs().max().item() / (y_eager.abs().max().item() + 1e-6))
    torch.cuda.synchronize()
    st = int(models["nvlink"].routed_experts.ep.nvlink.arena.status.item()) | int(torch.ops.tb200.gemm_status(True))
    st |= int(models["nvlink_exact"].routed_experts.ep.nvlink.arena.status.item())
    t = torch.tensor(res + [float(st)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        torch.save(t.cpu(), out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_expert_parallel_nvlink_matches_nccl(tmp_path):
    out = str(tmp_path / "ep.pt")
    run_distributed(_ep_nvlink, 2, out, backend="nccl")
    r = torch.load(out)
    assert r[-1] == 0, "a bounded wait expired"
    assert (r[:-1] < 3e-2).all(), r


def _cp_nvlink(rank, world, out_path):
    """Context-parallel KV exchange by peer loads against the NCCL collectives, forward and backward."""
    import torch.distributed as dist

    from torchtitan_b200.parallel.context_parallel import CPContext, _CPAllGather
    from torchtitan_b200.parallel.cp_nvlink import CPNvlink

    dev = torch.device("cuda", rank)
    group = dist.new_group(list(range(world)))
    nv = CPNvlink(group, dev, nbytes=8 << 20)
    torch.manual_seed(10 + rank)
    x = torch.randn(256, 8, 128, device=dev).bfloat16()
    got = nv.all_gather(x)
    want = torch.empty(world * 256, 8, 128, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(want, x, group=group)
    ok = torch.equal(got, want)
    full = torch.randn(world * 256, 8, 128, device=dev).bfloat16()
    rs = nv.reduce_scatter(full)
    ref = torch.empty(256, 8, 128, device=dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(ref, full.float(), group=group)
    ok = ok and torch.allclose(rs.float(), ref, atol=2e-2, rtol=2e-2)
    # through the autograd function both ways
    outs = []
    for transport in (None, nv):
        cp = CPContext(group=group, size=world, rank=rank, nvlink=transport)
        xi = x.clone().requires_grad_()
        y = _CPAllGather.apply(xi, cp)
        (y.float() * torch.arange(y.shape[0], device=dev)[:, None, None]).sum().backward()
        outs.append((y.detach(), xi.grad))
    ok = ok and torch.equal(outs[0][0], outs[1][0]) and torch.allclose(outs[0][1].float(), outs[1][1].float(), rtol=2e-2, atol=1.0)
    nv.check_status()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ok": int(flag.item())}, out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_context_parallel_nvlink_exchange(tmp_path):
    out = str(tmp_path / "cp.pt")
    run_distributed(_cp_nvlink, 2, out, backend="nccl")
    assert torch.load(out)["ok"] == 1


def _cp_flash(rank, world, mode, transport, out_path):
    """Context-parallel attention on the flash kernels (blocks with offsets, LSE merge) against the same
    kernels run on the whole sequence by one GPU: packed documents, a sliding window and sinks included."""
    import torch.distributed as dist

    from torchtitan_b200.models.common.attention import AttentionContext
    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.parallel.context_parallel import CPContext, cp_attention, shard_for_cp

    dev = torch.device("cuda", rank)
    T, Hq, Hkv, D = 2048, 4, 2, 128
    g = torch.Generator(device=dev).manual_seed(5)
    q = torch.randn(T, Hq, D, device=dev, generator=g).bfloat16()
    k = torch.randn(T, Hkv, D, device=dev, generator=g).bfloat16()
    v = torch.randn(T, Hkv, D, device=dev, generator=g).bfloat16()
    d_o = torch.randn(T, Hq, D, device=dev, generator=g).bfloat16()
    starts = torch.tensor([0, 300, 301, 1100, 1900], device=dev)
    pos = torch.arange(T, device=dev)
    doc_start = starts[torch.searchsorted(starts, pos, right=True) - 1]
    errs = []
    cp = CPContext(group=dist.group.WORLD, size=world, rank=rank, mode=mode)
    if transport == "nvlink":
        from torchtitan_b200.parallel.cp_nvlink import CPNvlink

        cp.nvlink = CPNvlink(dist.group.WORLD, dev, nbytes=16 << 20)
    idx = shard_for_cp(cp, pos, pos, pos)[3]
    for docs, window, use_sinks in ((False, None, False), (True, None, False), (True, 256, True)):
        kv_first = doc_start.int() if docs else None
        sinks_ref = torch.linspace(-1, 1, Hq, device=dev).requires_grad_() if use_sinks else None
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        ref = OF.attention(qf, kf, vf, causal=True, kv_first=kv_first, doc_ids=None if not docs else doc_start,
                           window=window, sinks=sinks_ref)
        ref.backward(d_o)
        ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
        ctx = AttentionContext(doc_ids=None if not docs else doc_start[idx].int(), q_pos=idx, cp=cp,
                               kv_first=None if not docs else doc_start[idx].int())
        sinks = sinks_ref.detach().clone().requires_grad_() if use_sinks else None
        out = cp_attention(ql, kl, vl, ctx, window=window, sinks=sinks)
        out.backward(d_o[idx])
        for got, want in ((out, ref[idx]), (ql.grad, qf.grad[idx]), (kl.grad, kf.grad[idx]), (vl.grad, vf.grad[idx])):
            errs.append((got.float() - want.float()).abs().max().item() / (want.float().abs().max().item() + 1e-6))
    torch.cuda.synchronize()
    st = int(torch.ops.tb200.flash_status(True))
    if cp.nvlink is not None:
        st |= int(cp.nvlink.arena.status.item())
    t = torch.tensor(errs + [float(st), float(OF.settings.library_fallbacks)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        torch.save(t.cpu(), out_path)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode,transport", [("allgather", "nccl"), ("ring", "nccl"), ("allgather", "nvlink"),
                                            ("ring", "nvlink")])
def test_context_parallel_attention_on_flash_kernels(tmp_path, mode, transport):
    out = str(tmp_path / "cpf.pt")
    run_distributed(_cp_flash, 2, mode, transport, out, backend="nccl")
    r = torch.load(out)
    assert r[-2] == 0, "a bounded wait expired"
    assert r[-1] == 0, "attention left the flash kernels"
    assert (r[:-2] < 3e-2).all(), r


def _graph_train(rank, world, graphs, out_path, folder):
    """A few trainer steps on 2 GPUs over the NVLink FSDP path, forward + backward eager or replayed from a
    CUDA graph (the flag barriers inside the graph must publish a fresh epoch on every replay)."""
    from torchtitan_b200.config import ConfigManager

    args = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "6",
            "--training.num_tokens_per_microbatch_per_dp_rank", "512", "--training.max_context_length", "256",
            "--debug.seed", "0", "--dump_folder", folder, "--debug.no-enable_structured_logging",
            "--checkpoint.no-enable", "--metrics.log_freq", "1", "--parallelism.fsdp_comm", "nvlink"]
    if graphs:
        args += ["--training.no-disable_cuda_graphs"]
    tr = ConfigManager().parse_args(args).build()
    assert tr.engines[0]._symm is not None
    losses = []
    it = tr.batch_generator(tr.dataloader)
    for _ in range(6):
        tr.step += 1
        tr.train_step(it)
        losses.append(tr._last_loss.detach().float().reshape(1).clone())
    if graphs:
        assert tr._graph_runner is not None and len(tr._graph_runner._graphs) >= 1
    t = torch.cat(losses)
    import torch.distributed as dist

    dist.all_reduce(t)
    tr.engines[0].check_status()
    if rank == 0:
        torch.save(t.cpu(), out_path)
    tr.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_cuda_graph_replay_over_nvlink_matches_eager(tmp_path):
    a, b = str(tmp_path / "eager.pt"), str(tmp_path / "graph.pt")
    run_distributed(_graph_train, 2, False, a, str(tmp_path / "e"), backend="nccl")
    run_distributed(_graph_train, 2, True, b, str(tmp_path / "g"), backend="nccl")
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=2e-2), (ra, rb)
    assert rb[-1] < rb[0]


def _pp_train(rank, world, pp, out_path, folder):
    """Trainer steps on GPUs with or without pipeline parallelism (same global batch: 2 microbatches per step)."""
    import torch.distributed as dist

    from torchtitan_b200.config import ConfigManager

    args = ["--module", "llama3", "--config", "llama3_debugmodel_hd128", "--training.steps", "4",
            "--training.num_tokens_per_microbatch_per_dp_rank", "512", "--training.max_context_length", "256",
            "--debug.seed", "0", "--dump_folder", folder, "--debug.no-enable_structured_logging",
            "--checkpoint.no-enable", "--metrics.log_freq", "1"]
    if pp > 1:
        args += ["--parallelism.pipeline_parallel_degree", str(pp), "--parallelism.pipeline_parallel_schedule", "1F1B",
                 "--parallelism.num_pp_microbatches", "2", "--parallelism.pipeline_parallel_layers_per_stage", "3"]
    else:
        args += ["--training.num_tokens_per_train_step", "1024"]
    tr = ConfigManager().parse_args(args).build()
    losses = []
    it = tr.batch_generator(tr.dataloader)
    for _ in range(4):
        tr.step += 1
        tr.train_step(it)
        losses.append(tr._last_loss.detach().float().reshape(1).clone())
    t = torch.cat(losses)
    if world > 1:
        dist.all_reduce(t)           # only the last stage holds the loss
    if rank == 0:
        torch.save(t.cpu(), out_path)
    tr.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pipeline_parallel_on_gpus_matches_single_gpu(tmp_path):
    """Two pipeline stages on two GPUs (1F1B, NCCL send / recv between stages, flash attention and tcgen05 GEMMs inside the
    stages) reproduce the single-GPU losses on the same microbatches."""
    a, b = str(tmp_path / "one.pt"), str(tmp_path / "pp.pt")
    run_distributed(_pp_train, 1, 1, a, str(tmp_path / "o"), backend="nccl")
    run_distributed(_pp_train, 2, 2, b, str(tmp_path / "p"), backend="nccl")
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=3e-2), (ra, rb)
