"""Experiments: RL losses / generator, Hugging Face backend, ForgeEngine, fault-tolerant replicas."""

import os
import time

import pytest
import torch

from tests.dist_utils import _free_port, run_distributed


# ---------------------------------------------------------------------------------------------
def test_grpo_loss_and_advantages():
    from torchtitan_b200.experiments.rl import dapo_loss, group_advantages, grpo_loss, token_logprobs

    torch.manual_seed(0)
    adv = group_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0]), group_size=2)
    assert torch.allclose(adv.view(3, 2).sum(1), torch.zeros(3), atol=1e-5) and adv[4] == 0
    logits = torch.randn(10, 7, requires_grad=True)
    toks = torch.randint(0, 7, (10,))
    lp, ent = token_logprobs(logits, toks)
    assert torch.allclose(lp.exp().detach(), torch.softmax(logits, -1)[torch.arange(10), toks].detach(), atol=1e-6)
    assert (ent > 0).all()
    mask = torch.tensor([0, 0, 1, 1, 1, 0, 1, 1, 1, 1.0])
    a = torch.where(torch.arange(10) < 5, torch.tensor(1.0), torch.tensor(-1.0))
    loss, stats = grpo_loss(lp, lp.detach(), a, mask, ref_logp=lp.detach() - 0.1, kl_coef=0.05)
    loss.backward()
    # on-policy: d loss / d logp = -adv / n on response tokens (+ the KL term's gradient), 0 elsewhere
    g = torch.autograd.grad(grpo_loss(token_logprobs(logits, toks)[0], lp.detach(), a, mask)[0], logits)[0]
    assert g[0].abs().max() == 0 and g[2].abs().max() > 0
    assert abs(stats["ratio_mean"] - 1.0) < 1e-6 and stats["kl"] > 0
    # clipping: a token whose ratio already exceeds 1 + eps with positive advantage gets no gradient
    lp2 = lp.detach().clone().requires_grad_()
    l2, _ = dapo_loss(lp2, lp.detach() - 1.0, torch.ones(10), mask, eps_low=0.2, eps_high=0.28)
    l2.backward()
    assert lp2.grad.abs().max() == 0


def test_generator_and_buffer_fold():
    from torchtitan_b200.experiments.rl import RolloutBuffer, SamplingGenerator, group_advantages, token_logprobs
    from torchtitan_b200.models import get_model_spec

    spec = get_model_spec("llama3", "debugmodel")
    spec.model.layers = spec.model.layers[:2]
    spec.model.n_layers = 2
    model = spec.model.build()
    model.init_states(seed=0)
    gen = SamplingGenerator(model, temperature=1.0, seed=1)
    prompt = torch.tensor([5, 9, 11])
    rolls = [gen.generate(prompt, 6) for _ in range(4)]
    assert all(r.response.numel() == 6 for r in rolls)
    for r, rew in zip(rolls, [1.0, 0.0, 0.5, 0.5]):
        r.reward = rew
    buf = RolloutBuffer()
    buf.add(rolls)
    adv = group_advantages(torch.tensor([r.reward for r in rolls]), 4)
    toks, pos, lab, old, a, mask = buf.fold(rolls, adv)
    assert toks.numel() == 4 * 9 and int(mask.sum()) == 24 and (pos == 0).sum() == 4
    logits = model(toks, pos)
    lp, _ = token_logprobs(logits, lab.clamp_min(0))
    # the behaviour policy is the current policy: recomputed log-probs match the recorded ones
    assert torch.allclose(lp[mask.bool()], old[mask.bool()], atol=1e-4)


def _tiny_llama(seed=0, layers=2):
    from torchtitan_b200.models import get_model_spec

    spec = get_model_spec("llama3", "debugmodel")
    spec.model.layers = spec.model.layers[:layers]
    spec.model.n_layers = layers
    model = spec.model.build()
    model.init_states(seed=seed)
    return spec, model


def test_cached_generator_matches_prefix_recomputation_and_weight_sync():
    from torchtitan_b200.experiments.rl import CachedGenerator, SamplingGenerator, WeightSync

    _, model = _tiny_llama(seed=0)
    prompt = torch.tensor([5, 9, 11, 4])
    slow = SamplingGenerator(model, temperature=0.0).generate(prompt, 8)
    fast = CachedGenerator(model, temperature=0.0).generate(prompt, 8)
    assert torch.equal(slow.response, fast.response)
    assert torch.allclose(slow.logprobs, fast.logprobs, atol=1e-4)
    # a generator with its own (stale) copy acts differently until the trainer's weights are pushed
    _, other = _tiny_llama(seed=1)
    gen = CachedGenerator(other, temperature=0.0)
    assert not torch.equal(gen.generate(prompt, 8).response, fast.response)
    sync = WeightSync()
    assert sync.push(model, gen) == 1 and gen.policy_version == 1
    assert torch.equal(gen.generate(prompt, 8).response, fast.response)


def test_rl_controller_improves_a_toy_reward():
    """DAPO with the cached generator on the debug model: the reward (share of answer tokens from the lower half of
    the vocabulary) rises within a few iterations; dynamic sampling drops groups without signal."""
    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.rl import CachedGenerator, RLConfig, RLController
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.trainer import Trainer

    spec, _ = _tiny_llama()
    cfg = Trainer.Config()
    cfg.training.mixed_precision_param = "float32"
    cfg.training.num_tokens_per_microbatch_per_dp_rank = 64
    cfg.training.max_context_length = 64
    pdims = ParallelDims(world_size=1)
    with torch.device("meta"):
        model = spec.model.build()
    eng = parallelize_decoder(model, pdims=pdims, job_config=cfg, device=torch.device("cpu"), seed=3)
    opt = OptimizersContainer(OptimizersContainer.Config(lr=2e-2, weight_decay=0.0), engines=[eng])
    reward = lambda prompt, resp: float((resp < 1024).float().mean())      # noqa: E731
    gen = CachedGenerator(model, temperature=1.0, seed=0)
    ctl = RLController(model, eng, opt, gen, reward, RLConfig(group_size=6, max_new_tokens=8, loss="dapo",
                                                               dynamic_sampling=True), pdims=pdims)
    prompts = [torch.tensor([3, 1, 4]), torch.tensor([1, 5, 9, 2])]
    hist = [ctl.step(prompts) for _ in range(12)]
    first = sum(h["reward_mean"] for h in hist[:3]) / 3
    last = sum(h["reward_mean"] for h in hist[-3:]) / 3
    assert last > first, (first, last)
    assert gen.policy_version == ctl.sync.version >= 1


def test_hf_backend_trains():
    transformers = pytest.importorskip("transformers")
    from torchtitan_b200.experiments.transformers_backend import HFCausalLM, hf_train_steps

    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    model = HFCausalLM(cfg)
    toks = torch.randint(0, 128, (33,))
    pos = torch.cat([torch.arange(20), torch.arange(12)])
    batch = (toks[:-1], pos, toks[1:])
    # packed documents do not see each other: the second document's logits equal a stand-alone run
    full = model(toks[:-1], pos)
    alone = model(toks[20:32], torch.arange(12))
    assert torch.allclose(full[20:], alone, atol=1e-4)
    losses = hf_train_steps(model, [batch] * 8, lr=3e-3)
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("module,flavor", [("deepseek_v3", "debugmodel"), ("qwen3_5", "debugmodel_moe"), ("muse_glimmer", "debugmodel"),
                                           ("kimi_k2_7", "debugmodel")])
def test_cached_generation_covers_latent_attention_and_recurrent_layers(module, flavor):
    """Incremental decoding equals prefix recomputation for latent attention (assembled keys / values cached), Gated
    DeltaNet layers (state matrix and convolution tails carried) and the gated-attention subclass, one sequence at a
    time and several sequences per pass in the engine."""
    import asyncio

    from torchtitan_b200.experiments.rl import GenerationEngine, SamplingConfig
    from torchtitan_b200.experiments.rl.generator import CachedGenerator, SamplingGenerator
    from torchtitan_b200.models import get_model_spec

    spec = get_model_spec(module, flavor)
    model = spec.model.build()
    model.init_states(seed=1)
    model.eval()
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn(p.shape, generator=g))
    prompts = [torch.randint(0, 2000, (n,), generator=g) for n in (70, 5)]
    want = [SamplingGenerator(model, temperature=0.0).generate(p, 10) for p in prompts]
    for p, w in zip(prompts, want):
        got = CachedGenerator(model, temperature=0.0).generate(p, 10)
        assert torch.equal(got.response, w.response) and torch.allclose(got.logprobs, w.logprobs, atol=1e-4)

    async def go():
        eng = GenerationEngine(GenerationEngine.Config(threaded=False), model=model)
        out = await asyncio.gather(*(eng.generate(p.tolist(), request_id=f"r{i}", sampling_config=SamplingConfig(
            temperature=0.0, max_tokens=10)) for i, p in enumerate(prompts)))
        await eng.close()
        return out

    for c, w in zip(asyncio.run(go()), want):
        assert c.token_ids == w.response.tolist() and torch.allclose(torch.tensor(c.token_logprobs), w.logprobs, atol=1e-4)


@pytest.mark.parametrize("module,flavor", [("llama3", "debugmodel_gqa"), ("gpt_oss", "debugmodel"), ("qwen3_5", "debugmodel")])
def test_cached_generation_matches_transformers_greedy(module, flavor):
    """Greedy decoding with the key / value cache (and, for GPT-OSS, a context longer than the sliding window, with
    sinks) produces the tokens ``transformers.generate`` produces on the same weights, as does the cache-free sampler."""
    transformers = pytest.importorskip("transformers")
    from torchtitan_b200.experiments.rl.generator import CachedGenerator, SamplingGenerator
    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.scripts.numerical_tests import checkpoint_state, hf_config_for, load_native_from_hf_state

    spec = get_model_spec(module, flavor)
    torch.manual_seed(0)
    hf = transformers.AutoModelForCausalLM.from_config(hf_config_for(module, spec.model)).float().eval()
    native = load_native_from_hf_state(spec, checkpoint_state(hf))
    prompt = torch.randint(0, 2048, (20,))
    with torch.no_grad():
        want = hf.generate(prompt[None], do_sample=False, max_new_tokens=50, pad_token_id=0)[0, 20:]
    for cls in (CachedGenerator, SamplingGenerator):
        got = cls(native, temperature=0.0).generate(prompt, 50).response
        assert torch.equal(got, want), (cls.__name__, int((got != want).sum()))


def test_forge_engine(tmp_path):
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.forge import ForgeEngine

    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.num_tokens_per_microbatch_per_dp_rank", "64",
        "--training.max_context_length", "64", "--training.mixed_precision_param", "float32", "--dump_folder", str(tmp_path),
        "--debug.no-enable_structured_logging", "--checkpoint.no-enable"])
    eng = ForgeEngine(cfg)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 2048, (65,), generator=g)
    losses = []
    for _ in range(4):
        losses.append(float(eng.forward_backward(ids[:-1], ids[1:])))
        eng.optimizer_step()
    assert losses[-1] < losses[0] and eng.step == 4
    with pytest.raises(RuntimeError):
        eng.train()
    eng.close()


def test_forge_example_trainer_matches_the_trainer_and_resumes(tmp_path):
    """The loop written on the engine's verbs (gradient accumulation over two microbatches) gives the Trainer's losses,
    and a second run resumes from the checkpoint the first one wrote."""
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.forge.example_train import main

    def args(folder, steps, ckpt):
        return ["--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", str(steps),
                "--training.num_tokens_per_microbatch_per_dp_rank", "64", "--training.max_context_length", "64",
                "--training.num_tokens_per_train_step", "128", "--training.mixed_precision_param", "float32",
                "--debug.seed", "0", "--dump_folder", str(folder), "--debug.no-enable_structured_logging",
                "--metrics.log_freq", "1"] + (["--checkpoint.enable", "--checkpoint.interval", "2"] if ckpt else
                                             ["--checkpoint.no-enable"])

    got = main(args(tmp_path / "a", 4, False))
    t = ConfigManager().parse_args(args(tmp_path / "b", 4, False)).build()
    want = []
    orig = t.metrics_processor.log

    def log(step, avg, mx, gn, extra_metrics=None):
        want.append(avg)
        return orig(step, avg, mx, gn, extra_metrics=extra_metrics)

    t.metrics_processor.log = log
    t.train()
    t.close()
    assert torch.allclose(torch.tensor(got), torch.tensor(want), atol=1e-5), (got, want)
    first = main(args(tmp_path / "c", 2, True))
    rest = main(args(tmp_path / "c", 4, True))          # resumes at step 2
    assert len(first) == 2 and len(rest) == 2
    assert torch.allclose(torch.tensor(first + rest), torch.tensor(got), atol=1e-5), (first, rest, got)


# ---------------------------------------------------------------------------------------------
def _replica(rid, n, port, die_at, out):
    """A replica trains a least-squares model; replica ``n - 1`` stops between steps at ``die_at``."""
    from datetime import timedelta

    from torch.distributed import TCPStore

    from torchtitan_b200.experiments.ft import FTManager

    store = TCPStore("127.0.0.1", port, world_size=n, is_master=(rid == 0), timeout=timedelta(seconds=60),
                     wait_for_workers=True)
    mgr = FTManager(store, rid, n, heartbeat_timeout=1.0, quorum_timeout=5.0)
    torch.manual_seed(0)
    w = torch.zeros(4, requires_grad=True)
    target = torch.tensor([1.0, -2.0, 3.0, 0.5])
    g = torch.Generator().manual_seed(100 + rid)
    hist = []
    for step in range(8):
        if rid == n - 1 and step == die_at:
            return                                    # leaves between steps, nothing in flight
        q = mgr.start_quorum(step)
        x = torch.randn(16, 4, generator=g)
        loss = ((x @ w - x @ target) ** 2).mean()
        (grad,) = torch.autograd.grad(loss, w)
        mgr.allreduce([grad])
        if mgr.should_commit():
            with torch.no_grad():
                w -= 0.1 * grad
        hist.append((step, list(q.members), float(loss)))
    torch.save({"w": w.detach(), "hist": hist}, out.format(rid))
    if rid == 0:
        time.sleep(1.0)                               # keep the store alive until the others have finished


def test_replica_loss_is_detected_and_training_continues(tmp_path):
    import torch.multiprocessing as mp

    n, port = 3, _free_port()
    out = str(tmp_path / "r{}.pt")
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_replica, args=(r, n, port, 3, out)) for r in range(n)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    a, b = torch.load(out.format(0)), torch.load(out.format(1))
    assert not os.path.exists(out.format(2))
    assert [m for _, m, _ in a["hist"]] == [[0, 1, 2]] * 3 + [[0, 1]] * 5
    assert torch.equal(a["w"], b["w"])               # survivors stay in lock-step
    assert a["hist"][-1][2] < a["hist"][0][2]


def test_diloco_outer_step():
    from torchtitan_b200.experiments.ft import DiLoCo, FTManager

    class _Store(dict):
        def set(self, k, v):
            self[k] = v if isinstance(v, bytes) else str(v).encode()

        def get(self, k):
            return self[k]

        def check(self, keys):
            return all(k in self for k in keys)

    mgr = FTManager(_Store(), 0, 1)
    p = torch.nn.Parameter(torch.ones(3))
    algo = DiLoCo(mgr, [p], sync_every=2, outer_lr=1.0, momentum=0.0)
    with torch.no_grad():
        p -= 0.5
    assert not algo.step()
    with torch.no_grad():
        p -= 0.25
    assert algo.step()
    # pseudo-gradient = global - local = 0.75; outer SGD with lr 1 moves the global weights onto the local ones
    assert torch.allclose(p.detach(), torch.full((3,), 0.25))


def _hf_engine(rank, world, reshard, out_path):
    import transformers

    from torchtitan_b200.experiments.transformers_backend import HFCausalLM, hf_engine_train_steps, parallelize_hf
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.trainer import Trainer

    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                   tie_word_embeddings=False)
    torch.manual_seed(0)
    model = HFCausalLM(cfg)
    job = Trainer.Config()
    job.training.mixed_precision_param = "float32"
    job.parallelism.fsdp_reshard_after_forward = reshard
    pdims = ParallelDims(world_size=world, rank=rank).build()
    eng = parallelize_hf(model, pdims=pdims, job_config=job, device=torch.device("cpu"))
    g = torch.Generator().manual_seed(1)
    batches = []
    for s in range(4):
        per_rank = []
        for r in range(2):
            toks = torch.randint(0, 128, (33,), generator=g)
            per_rank.append((toks[:-1], torch.arange(32), toks[1:]))
        batches.append(per_rank)
    mine = [b[rank] for b in batches] if world == 2 else None
    if world == 2:
        losses = hf_engine_train_steps(model, eng, mine, pdims=pdims, lr=3e-3)
    else:   # one rank sees both sequences of a step as one packed batch
        packed = [(torch.cat([a[0], b[0]]), torch.cat([a[1], b[1]]), torch.cat([a[2], b[2]])) for a, b in batches]
        losses = hf_engine_train_steps(model, eng, packed, pdims=pdims, lr=3e-3)
    if rank == 0:
        torch.save(torch.tensor(losses), out_path)


def test_hf_model_on_the_sharded_engine(tmp_path):
    """A Hugging Face Llama under the flat-buffer FSDP engine: 2 ranks (resident and sharded layout) reproduce the
    single-rank losses on the same global batch."""
    pytest.importorskip("transformers")
    from tests.dist_utils import run_distributed

    outs = {}
    for name, world, reshard in (("one", 1, "never"), ("resident", 2, "never"), ("sharded", 2, "always")):
        path = str(tmp_path / f"{name}.pt")
        run_distributed(_hf_engine, world, reshard, path)
        outs[name] = torch.load(path)
    assert torch.allclose(outs["one"], outs["resident"], atol=2e-4), outs
    assert torch.allclose(outs["one"], outs["sharded"], atol=2e-4), outs
    assert outs["one"][-1] < outs["one"][0]


def _hf_tp(rank, world, tp, out_path):
    import transformers

    from torchtitan_b200.experiments.transformers_backend import HFCausalLM, hf_engine_train_steps, parallelize_hf
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.trainer import Trainer

    cfg = transformers.Qwen3Config(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=64,
                                   tie_word_embeddings=False)
    torch.manual_seed(0)
    model = HFCausalLM(cfg)
    job = Trainer.Config()
    job.training.mixed_precision_param = "float32"
    pdims = ParallelDims(world_size=world, rank=rank, tp=tp).build()
    eng = parallelize_hf(model, pdims=pdims, job_config=job, device=torch.device("cpu"))
    if tp > 1:
        q = model.hf.model.layers[0].self_attn.q_proj
        assert q.weight.shape == (32 // tp, 32) and q.weight._tp_slices[0] == 0
        assert model.hf.model.layers[0].mlp.down_proj.weight.shape == (32, 64 // tp)
    g = torch.Generator().manual_seed(1)
    batches = []
    for s in range(4):
        per_rank = []
        for r in range(2):
            toks = torch.randint(0, 128, (33,), generator=g)
            per_rank.append((toks[:-1], torch.arange(32), toks[1:]))
        batches.append(per_rank)
    if pdims.dp_degree == 2:
        mine = [b[pdims.dp_rank] for b in batches]
    else:   # one data rank sees both sequences of a step as one packed batch
        mine = [(torch.cat([a[0], b[0]]), torch.cat([a[1], b[1]]), torch.cat([a[2], b[2]])) for a, b in batches]
    losses = hf_engine_train_steps(model, eng, mine, pdims=pdims, lr=3e-3)
    gn = float(sum((u.master.double() ** 2).sum() for u in eng.units))
    if rank == 0:
        torch.save(torch.tensor(losses + [gn]), out_path)


def test_hf_model_tensor_parallel(tmp_path):
    """A Hugging Face Qwen3 (per-head q / k norms) with its projections split over tp 2, alone and under dp 2 x tp 2:
    the losses of the single-rank run."""
    pytest.importorskip("transformers")
    from tests.dist_utils import run_distributed

    outs = {}
    for name, world, tp in (("one", 1, 1), ("tp2", 2, 2), ("dp2tp2", 4, 2)):
        path = str(tmp_path / f"{name}.pt")
        run_distributed(_hf_tp, world, tp, path)
        outs[name] = torch.load(path)
    assert torch.allclose(outs["one"][:-1], outs["tp2"][:-1], atol=2e-4), outs
    assert torch.allclose(outs["one"][:-1], outs["dp2tp2"][:-1], atol=2e-4), outs


def _hf_pp(rank, world, out_path):
    import transformers

    from torchtitan_b200.experiments.transformers_backend import (HFCausalLM, hf_engine_train_steps, hf_pipeline_train_steps,
                                                                  parallelize_hf, pipeline_hf)
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.trainer import Trainer

    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                   tie_word_embeddings=False)
    torch.manual_seed(0)
    model = HFCausalLM(cfg)
    job = Trainer.Config()
    job.training.mixed_precision_param = "float32"
    job.parallelism.pipeline_parallel_schedule = "1F1B"
    job.parallelism.num_pp_microbatches = 2
    g = torch.Generator().manual_seed(1)
    steps = []
    for s in range(4):
        toks = torch.randint(0, 128, (2, 33), generator=g)
        steps.append((toks[:, :-1].contiguous(), torch.arange(32).expand(2, 32).contiguous(), toks[:, 1:].contiguous()))
    if world == 1:
        pdims = ParallelDims(world_size=1, rank=0).build()
        eng = parallelize_hf(model, pdims=pdims, job_config=job, device=torch.device("cpu"))
        packed = [(t.reshape(-1), p.reshape(-1), l.reshape(-1)) for t, p, l in steps]
        losses = hf_engine_train_steps(model, eng, packed, pdims=pdims, lr=3e-3)
    else:
        pdims = ParallelDims(world_size=world, rank=rank, pp=2).build()
        sched, stage, eng, first, last = pipeline_hf(model, pdims=pdims, job_config=job, device=torch.device("cpu"))
        assert (stage.embed_tokens is not None) == (rank == 0) and (stage.lm_head is not None) == (rank == 1)
        assert len(stage.layers) in (2, 3)
        losses = hf_pipeline_train_steps(sched, eng, steps, pdims=pdims, has_first=first, has_last=last, lr=3e-3)
    if rank == 0:
        torch.save(torch.tensor(losses), out_path)


def test_hf_model_pipeline_parallel(tmp_path):
    """A Hugging Face Llama split into two pipeline stages (1F1B, two microbatches, each stage under the sharded
    engine) reproduces the single-rank losses on the same batches."""
    pytest.importorskip("transformers")
    from tests.dist_utils import run_distributed

    a, b = str(tmp_path / "one.pt"), str(tmp_path / "pp.pt")
    run_distributed(_hf_pp, 1, a)
    run_distributed(_hf_pp, 2, b)
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=2e-4), (ra, rb)


def test_graph_trainer_passes_map_to_engine_settings(tmp_path):
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.graph_trainer import GraphTrainer, apply_passes

    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.num_tokens_per_microbatch_per_dp_rank", "64",
        "--training.max_context_length", "64", "--training.steps", "2", "--training.mixed_precision_param", "float32",
        "--dump_folder", str(tmp_path), "--debug.no-enable_structured_logging"])
    done = apply_passes(cfg, ["fsdp_reshard", "async_tp", "ep_overlap", "full_remat", "regional_inductor"])
    assert done == ["fsdp_reshard", "async_tp", "ep_overlap", "full_remat"]
    assert cfg.parallelism.fsdp_reshard_after_forward == "always" and cfg.parallelism.tp_comm == "nvlink"
    assert cfg.parallelism.ep_comm == "nvlink" and cfg.activation_checkpoint.mode == "full"
    with pytest.raises(ValueError):
        apply_passes(cfg, ["no_such_pass"])
    with pytest.raises(ValueError):
        apply_passes(cfg, ["cudagraph", "cpu_offload"])
    cfg.training.disable_cuda_graphs = True
    cfg.activation_checkpoint.cpu_offload = False
    t = GraphTrainer(cfg, passes=["selective_remat", "fsdp_overlap"])
    t.train()
    assert t.step == 2 and t.applied_passes == ["selective_remat", "fsdp_overlap"]
    t.close()


def _ft_replica(rid, n, port, die_at, out, folder):
    """A replica group = one single-process trainer; replica ``n - 1`` leaves between steps at ``die_at``."""
    from datetime import timedelta

    from torch.distributed import TCPStore

    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.ft import FaultToleranceConfig, FaultTolerantTrainer

    store = TCPStore("127.0.0.1", port, world_size=n, is_master=(rid == 0), timeout=timedelta(seconds=60),
                     wait_for_workers=True)
    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.num_tokens_per_microbatch_per_dp_rank", "64",
        "--training.max_context_length", "64", "--training.mixed_precision_param", "float32", "--debug.seed", "0",
        "--dump_folder", f"{folder}/r{rid}", "--debug.no-enable_structured_logging", "--checkpoint.no-enable",
        "--dataloader.seed", str(10 + rid), "--metrics.log_freq", "100"])
    ft = FaultToleranceConfig(enable=True, replica_id=rid, group_size=n, heartbeat_timeout_s=4.0, quorum_timeout_s=12.0)
    t = FaultTolerantTrainer(cfg, fault_tolerance=ft, store=store)
    it = t.batch_generator(t.dataloader)
    members, losses = [], []
    for step in range(6):
        if rid == n - 1 and step == die_at:
            return                                          # leaves between steps
        t.step += 1
        t.train_step(it)
        t.checkpointer.save(t.step)
        members.append(list(t.manager.members))
        losses.append(float(t._last_loss))
    w = torch.cat([u.master for e in t.engines for u in e.units])
    torch.save({"members": members, "losses": losses, "w": w, "skipped": t.optimizers.skipped}, out.format(rid))
    assert os.path.exists(os.path.join(cfg.dump_folder, f"ft-replica-{rid}", "dataloader.pt"))
    if rid == 0:
        time.sleep(1.0)
    t.close()


def test_fault_tolerant_trainer_survives_a_lost_replica(tmp_path):
    """Two replica groups average gradients through the FT manager; one leaves after step 3, the other goes on alone
    (its quorum shrinks) and keeps training."""
    import torch.multiprocessing as mp

    from tests.dist_utils import _free_port

    port = _free_port()
    out = str(tmp_path / "ft{}.pt")
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_ft_replica, args=(r, 2, port, 3, out, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    r0 = torch.load(out.format(0))
    assert r0["members"][:3] == [[0, 1]] * 3 and r0["members"][-1] == [0]
    assert all(l == l for l in r0["losses"]) and r0["skipped"] == 0


def test_fragment_llm_covers_every_parameter_once():
    from torchtitan_b200.experiments.ft import fragment_llm

    _, model = _tiny_llama(layers=4)
    frags = fragment_llm(model, 3)
    ids = [id(p) for f in frags for p in f]
    assert len(ids) == len(set(ids)) == len(list(model.parameters())) and len(frags) >= 2


@pytest.mark.parametrize("family", ["qwen3_moe", "deepseek_v3"])
def test_hf_backend_native_moe_replacement(family):
    """The HF model with its expert blocks swapped for the native MoE layer gives the HF model's logits (softmax
    top-k with renormalisation; sigmoid routing with groups, selection bias, scaling and shared experts), trains,
    and the trained weights go back into the HF blocks."""
    transformers = pytest.importorskip("transformers")
    from torchtitan_b200.experiments.transformers_backend import HFCausalLM, hf_train_steps
    from torchtitan_b200.experiments.transformers_backend.moe_replacement import (NativeMoEAdapter, probe_hf_moe_block,
                                                                                  restore_hf_moe_state, swap_native_moe)

    if family == "qwen3_moe":
        cfg = transformers.Qwen3MoeConfig(vocab_size=128, hidden_size=32, intermediate_size=64, moe_intermediate_size=16,
                                          num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                                          num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
                                          mlp_only_layers=[], max_position_embeddings=64)
    else:
        cfg = transformers.DeepseekV3Config(vocab_size=128, hidden_size=32, intermediate_size=64, moe_intermediate_size=16,
                                            num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                                            n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=3, n_group=4,
                                            topk_group=2, routed_scaling_factor=2.5, norm_topk_prob=True,
                                            first_k_dense_replace=1, q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8,
                                            qk_rope_head_dim=8, v_head_dim=8, max_position_embeddings=64)
    torch.manual_seed(0)
    model = HFCausalLM(cfg)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.2)                               # the default init leaves routing nearly uniform
        for name, b in model.named_buffers():
            if name.endswith("e_score_correction_bias"):
                b.normal_(0, 0.1)
    toks = torch.randint(0, 128, (41,))
    pos = torch.cat([torch.arange(25), torch.arange(16)])
    with torch.no_grad():
        want = model(toks, pos)
    n_moe = sum(1 for layer in model.hf.model.layers if hasattr(layer.mlp, "experts"))
    info = probe_hf_moe_block(next(layer.mlp for layer in model.hf.model.layers if hasattr(layer.mlp, "experts")))
    assert info["num_experts"] == 8 and info["score_func"] == ("softmax" if family == "qwen3_moe" else "sigmoid")
    assert swap_native_moe(model) == n_moe > 0 and swap_native_moe(model) == 0
    assert sum(isinstance(layer.mlp, NativeMoEAdapter) for layer in model.hf.model.layers) == n_moe
    with torch.no_grad():
        got = model(toks, pos)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), float((got - want).abs().max())
    batch = (toks[:-1], pos[:-1], toks[1:])
    losses = hf_train_steps(model, [batch] * 6, lr=3e-3)
    assert losses[-1] < losses[0]
    with torch.no_grad():
        trained = model(toks, pos)
    assert restore_hf_moe_state(model) == n_moe
    assert not any(isinstance(layer.mlp, NativeMoEAdapter) for layer in model.hf.model.layers)
    with torch.no_grad():
        back = model(toks, pos)
    assert torch.allclose(back, trained, atol=2e-4, rtol=1e-4) and not torch.allclose(back, want, atol=1e-3)


def test_ft_config_registry_builds_the_fault_tolerant_trainer(tmp_path):
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.ft import config_registry as reg

    assert reg.llama3_ft_debugmodel_diloco().fault_tolerance.semi_sync_method == "diloco"
    cfg = ConfigManager().parse_args([
        "--module", "ft", "--config", "llama3_ft_debugmodel", "--fault_tolerance.replica_id", "1",
        "--fault_tolerance.no-enable", "--training.steps", "1", "--training.num_tokens_per_microbatch_per_dp_rank", "64",
        "--training.max_context_length", "64", "--training.mixed_precision_param", "float32", "--dump_folder", str(tmp_path),
        "--debug.no-enable_structured_logging", "--checkpoint.no-enable"])
    assert cfg.fault_tolerance.replica_id == 1 and cfg.fault_tolerance.group_size == 2 and cfg.model.flavor == "debugmodel"
    t = cfg.build()
    assert type(t).__name__ == "FaultTolerantTrainer" and t.manager is None       # disabled: a plain trainer
    t.train()
    t.close()


def _hf_train_entry(rank, world, out_path, extra):
    from torchtitan_b200.experiments.transformers_backend.train import main

    extra = list(extra)
    steps = "5"
    if "--steps-override" in extra:
        i = extra.index("--steps-override")
        steps = extra[i + 1]
        del extra[i:i + 2]
    losses = main(["--steps", steps, "--training.num_tokens_per_microbatch_per_dp_rank", "128", "--training.max_context_length",
                   "64", "--training.mixed_precision_param", "float32", "--optimizer.lr", "5e-3", "--lr_scheduler.warmup_steps",
                   "1", "--debug.seed", "1", "--debug.no-enable_structured_logging", *extra])
    if rank == 0:
        torch.save(losses, out_path)


def test_hf_backend_train_entry(tmp_path):
    """The backend's command line: registered debug architectures, native MoE swap, data and tensor parallelism.  Two
    tensor-parallel ranks see the data of the single-rank run and reproduce its losses."""
    import math

    pytest.importorskip("transformers")
    got = {}
    for name, world, extra in [("one", 1, ("--hf-model", "debug_llama")),
                               ("tp2", 2, ("--hf-model", "debug_llama", "--parallelism.tensor_parallel_degree", "2")),
                               ("moe", 1, ("--hf-model", "debug_deepseek_v3", "--native-moe", "--steps-override", "3"))]:
        out = str(tmp_path / f"{name}.pt")
        run_distributed(_hf_train_entry, world, out, extra)
        got[name] = torch.load(out)
        assert len(got[name]) in (3, 5) and all(math.isfinite(x) for x in got[name]), (name, got[name])
    assert torch.allclose(torch.tensor(got["one"]), torch.tensor(got["tp2"]), atol=2e-3), (got["one"], got["tp2"])
    assert got["one"][0] != got["one"][-1]


def test_compile_passes_from_the_command_line():
    """``--compile.passes`` on the ordinary trainer's command line folds the graph trainer's pass names into the
    config at validation; unknown names are refused."""
    from torchtitan_b200.config import ConfigManager

    cfg = ConfigManager().parse_args(["--module", "llama3", "--config", "llama3_debugmodel", "--compile.passes",
                                      "full_remat,fsdp_reshard,ep_overlap,regional_inductor"])
    assert cfg.activation_checkpoint.mode == "full" and cfg.parallelism.fsdp_reshard_after_forward == "always"
    assert cfg.parallelism.ep_comm == "nvlink"
    with pytest.raises(ValueError, match="unknown graph_trainer pass"):
        ConfigManager().parse_args(["--module", "llama3", "--config", "llama3_debugmodel", "--compile.passes", "nonsense"])
