"""Context parallel attention (all-gather and ring) equals single-device causal attention."""

import pytest
import torch

from tests.dist_utils import run_distributed


def _cp_fn(rank, world, mode, with_docs, out_path, window=None, use_sinks=False, balancer="headtail"):
    import torch.distributed as dist

    from torchtitan_b200.models.common.attention import AttentionContext
    from torchtitan_b200.ops import functional as OF
    from torchtitan_b200.parallel.context_parallel import CPContext, cp_attention, shard_for_cp, unshard_from_cp

    torch.manual_seed(0)
    T, Hq, Hkv, D = 32, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    g = torch.randn(T, Hq, D)
    doc = None
    if with_docs:
        doc = torch.tensor([1] * 10 + [2] * 15 + [3] * 7, dtype=torch.int32)
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    sinks_ref = torch.tensor([0.3, -0.5, 1.0, 0.0]).requires_grad_() if use_sinks else None
    ref = OF.attention(qf, kf, vf, doc_ids=doc, window=window, sinks=sinks_ref)
    ref.backward(g)

    cp = CPContext(group=dist.group.WORLD, size=world, rank=rank, mode=mode, load_balancer=balancer)
    if balancer == "ptrr":
        from torchtitan_b200.parallel.context_parallel import ptrr_assignment

        positions = torch.cat([torch.arange(10), torch.arange(15), torch.arange(7)]) if with_docs else torch.arange(T)
        cp.assignment = ptrr_assignment(positions, world, chunks_per_rank=4)
        assert sorted(c for a in cp.assignment for c in a) == list(range(4 * world))
    idx = shard_for_cp(cp, torch.arange(T), torch.arange(T), torch.arange(T))[3]
    ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
    ctx = AttentionContext(doc_ids=None if doc is None else doc[idx], q_pos=idx, cp=cp)
    sinks = sinks_ref.detach().clone().requires_grad_() if use_sinks else None
    out = cp_attention(ql, kl, vl, ctx, window=window, sinks=sinks)
    out.backward(g[idx])
    ok = torch.allclose(out, ref[idx].detach(), atol=1e-5)
    if use_sinks:
        gs = sinks.grad.clone()
        dist.all_reduce(gs)
        ok = ok and torch.allclose(gs, sinks_ref.grad, atol=1e-5)
    ok = ok and torch.allclose(ql.grad, qf.grad[idx], atol=1e-5)
    ok = ok and torch.allclose(kl.grad, kf.grad[idx], atol=1e-5)
    ok = ok and torch.allclose(vl.grad, vf.grad[idx], atol=1e-5)
    full = unshard_from_cp(cp, out.detach())
    ok = ok and torch.allclose(full, ref.detach(), atol=1e-5)
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save(flag, out_path)


@pytest.mark.parametrize("mode", ["allgather", "ring"])
@pytest.mark.parametrize("with_docs", [False, True])
def test_cp_attention_matches_full(tmp_path, mode, with_docs):
    out = str(tmp_path / "cp.pt")
    run_distributed(_cp_fn, 2, mode, with_docs, out)
    assert float(torch.load(out)) == 1.0


@pytest.mark.parametrize("mode", ["allgather", "ring"])
def test_cp_attention_window_documents_and_sinks(tmp_path, mode):
    out = str(tmp_path / "cpw.pt")
    run_distributed(_cp_fn, 2, mode, True, out, 6, True)
    assert float(torch.load(out)) == 1.0


@pytest.mark.parametrize("mode", ["allgather", "ring"])
def test_cp_attention_with_ptrr_balancer(tmp_path, mode):
    out = str(tmp_path / "cpp.pt")
    run_distributed(_cp_fn, 2, mode, True, out, None, False, "ptrr")
    assert float(torch.load(out)) == 1.0


def test_ptrr_assignment_balances_uneven_documents():
    from torchtitan_b200.parallel.context_parallel import ptrr_assignment

    # one long document followed by many short ones: head-tail pairing would overload the ranks holding the long one
    pos = torch.cat([torch.arange(4096)] + [torch.arange(64)] * 64)
    a = ptrr_assignment(pos, 4, chunks_per_rank=8)
    work = (pos.double() + 1).view(32, -1).sum(1)
    loads = [sum(float(work[c]) for c in chunks) for chunks in a]
    assert max(loads) / min(loads) < 1.15
    assert all(len(c) == 8 for c in a)


def test_headtail_chunks():
    from torchtitan_b200.parallel.context_parallel import CPContext, cp_chunk_ids

    cp = CPContext(group=None, size=4, rank=1)
    assert cp_chunk_ids(cp) == [1, 6]
    assert sorted(c for r in range(4) for c in cp_chunk_ids(cp, r)) == list(range(8))
