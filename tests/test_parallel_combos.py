"""Combinations of parallelisms on CPU / gloo: HSDP (replicate x shard), and pipeline stages whose
parameters use the sharded layout.  Reference cases: tests/integration_tests/features.py (ddp / hsdp / pp+fsdp)."""

import pytest
import torch

from tests.dist_utils import run_distributed


def _run(rank, world, extra, out_path, global_tokens, module="llama3", config="llama3_debugmodel"):
    from torchtitan_b200.config import ConfigManager

    args = ["--module", module, "--config", config, "--training.steps", "3",
            "--training.num_tokens_per_microbatch_per_dp_rank", "64", "--training.max_context_length", "64",
            "--training.mixed_precision_param", "float32", "--debug.seed", "0", "--dump_folder", out_path + "_d",
            "--debug.no-enable_structured_logging", "--metrics.log_freq", "1",
            "--training.num_tokens_per_train_step", str(global_tokens)] + list(extra)
    t = ConfigManager().parse_args(args).build()
    losses = []
    orig = t.metrics_processor.log

    def log(step, avg, mx, gn, extra_metrics=None):
        losses.append((avg, gn))
        return orig(step, avg, mx, gn, extra_metrics=extra_metrics)

    t.metrics_processor.log = log
    t.train()
    if rank == 0:
        torch.save(torch.tensor(losses), out_path)
    t.close()


def test_hsdp_matches_fsdp(tmp_path):
    """dp_replicate 2 x dp_shard 2 trains like dp_shard 4: same global batch, gradients summed over both axes."""
    a, b = str(tmp_path / "fsdp.pt"), str(tmp_path / "hsdp.pt")
    run_distributed(_run, 4, ["--parallelism.data_parallel_shard_degree", "4"], a, 256, timeout=400)
    run_distributed(_run, 4, ["--parallelism.data_parallel_replicate_degree", "2",
                              "--parallelism.data_parallel_shard_degree", "2"], b, 256, timeout=400)
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=2e-4), (ra, rb)


def test_pipeline_stages_with_sharded_parameters(tmp_path):
    """pp 2 x dp_shard 2: stages that gather their units per use and reduce-scatter every microbatch
    (fsdp_reshard_after_forward = always) give the losses of stages with resident parameters."""
    pp = ["--parallelism.pipeline_parallel_degree", "2", "--parallelism.pipeline_parallel_schedule", "1F1B",
          "--parallelism.num_pp_microbatches", "2", "--parallelism.data_parallel_shard_degree", "2"]
    a, b = str(tmp_path / "never.pt"), str(tmp_path / "always.pt")
    run_distributed(_run, 4, pp + ["--parallelism.fsdp_reshard_after_forward", "never"], a, 256, timeout=400)
    run_distributed(_run, 4, pp + ["--parallelism.fsdp_reshard_after_forward", "always"], b, 256, timeout=400)
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=1e-5), (ra, rb)


def test_expert_tensor_parallel_matches_data_parallel(tmp_path):
    """Expert tensor parallelism (tp 2, expert parallelism off: w1 / w3 split over the hidden dimension, w2 over its
    input, the layer's output a partial sum reduced over tp; reference plan: models/common/moe_sharding.py:50-68)
    and tp 2 x ep 2 (experts split over ep, tokens stay split over tp) train a mixture-of-experts model like two
    data-parallel ranks on the same global batch (data-parallel degree 2 in all three)."""
    moe = ("qwen3", "qwen3_moe_tiny")
    a, b, c = (str(tmp_path / n) for n in ("dp.pt", "etp.pt", "tp_ep.pt"))
    run_distributed(_run, 2, ["--parallelism.data_parallel_shard_degree", "2"], a, 256, *moe, timeout=400)
    run_distributed(_run, 4, ["--parallelism.tensor_parallel_degree", "2", "--parallelism.data_parallel_shard_degree", "2"],
                    b, 256, *moe, timeout=400)
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=3e-4), (ra, rb)
    run_distributed(_run, 4, ["--parallelism.tensor_parallel_degree", "2", "--parallelism.expert_parallel_degree", "2",
                              "--parallelism.data_parallel_shard_degree", "2"], c, 256, *moe, timeout=400)
    rc = torch.load(c)
    assert torch.allclose(ra, rc, atol=3e-4), (ra, rc)


def test_local_tensor_mode_validates_the_sharding_plan():
    """comm.mode = local_tensor: one process walks over 8 emulated ranks (dp_shard 4 x tp 2) and checks that their
    shards tile every parameter exactly once; a plan with a hole is reported."""
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.parallel import local_plan

    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.num_tokens_per_microbatch_per_dp_rank", "64",
        "--training.max_context_length", "64", "--parallelism.tensor_parallel_degree", "2", "--comm.mode", "local_tensor"])
    covered = local_plan.validate_plan(cfg, world=8)
    assert any("wqkv" in k for k in covered) and all(v > 0 for v in covered.values())
    orig = local_plan._rank_plan

    def broken(config, world, rank):
        owned, total = orig(config, world, rank)
        if rank == 3:
            owned.pop(next(iter(owned)))
        return owned, total

    local_plan._rank_plan = broken
    try:
        with pytest.raises(RuntimeError, match="does not tile"):
            local_plan.validate_plan(cfg, world=8)
    finally:
        local_plan._rank_plan = orig


def test_declarative_sharding_contracts_drive_the_slices():
    """Every tensor-parallel module declares its contract (parameter placements, input / output placement pairs);
    the slices the modules hold are cut from those declarations, and the boundary collectives follow from the
    (source, destination) pairs.  Reference: protocols/sharding.py:69-168, models/common/decoder_sharding.py."""
    from types import SimpleNamespace

    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.models.common.layers import TPContext
    from torchtitan_b200.parallel import sharding as shd

    assert shd.redistribution(shd.Shard(0), shd.Replicate()) == "all_gather_rows"
    assert shd.redistribution(shd.Partial(), shd.Shard(0)) == "reduce_scatter_rows"
    assert shd.redistribution(shd.Partial(), shd.Replicate()) == "all_reduce"
    assert shd.redistribution(shd.Replicate(), shd.Replicate()) == "copy"
    with pytest.raises(ValueError):
        shd.redistribution(shd.Shard(1), shd.Replicate())
    with pytest.raises(ValueError):
        shd.SpmdLayout(model_parallel=shd.Shard(0))
    lay = shd.SpmdLayout(tp=shd.Shard(0), dp_shard=shd.Shard(0))
    assert shd.resolve_placements(lay, [("dp_shard", 4), ("cp", 2), ("tp", 1)]) == (shd.Shard(0), shd.Replicate(), shd.Replicate())

    for module, flavor in (("llama3", "debugmodel"), ("qwen3", "debugmodel_moe_tiny")):
        with torch.device("meta"):
            model = get_model_spec(module, flavor).model.build()
        tp = TPContext(group=None, size=2, rank=1)
        par = SimpleNamespace(tensor_parallel_degree=2, disable_sequence_parallel=False, tp_comm="nccl", enable_loss_parallel=True)
        model.tok_embeddings.shard_(tp)
        for blk in model.layers.values():
            blk.attention.shard_(tp)
            if blk.feed_forward is not None:
                blk.feed_forward.shard_(tp)
            if blk.moe is not None:
                blk.moe.shard_tp_(tp)
        model.lm_head.shard_("colwise", tp)
        table = shd.sharding_table(model)
        assert table["tok_embeddings"]["state"]["weight"] == {"tp": "S(0)"}
        assert table["tok_embeddings"]["out"] == [{"tp": "P"}, {"tp": "S(0)"}]
        assert table["layers.0.attention.wo"]["state"]["weight"] == {"tp": "S(1)"}
        assert table["layers.0.attention_norm"]["state"]["weight"] == {"tp": "R"}
        if module == "qwen3":
            ex = table["layers.0.moe.routed_experts.inner_experts"]
            assert ex["state"]["w2_EDF"] == {"tp": "S(2)"} and ex["out"][0] == {"tp": "P"}
        n = shd.check_against_slices(model, "tp")
        assert n > 10
        # a slice that contradicts the declaration is reported
        wo = model.layers["0"].attention.wo
        wo.weight._tp_slices = (0,) + wo.weight._tp_slices[1:]
        with pytest.raises(RuntimeError, match="declared S\\(1\\)"):
            shd.check_against_slices(model, "tp")


def test_tensor_parallel_without_sequence_parallel_matches_single_rank(tmp_path):
    """tp 2 with replicated activations between the blocks: the block norms then hold their complete gradient on every
    rank (not summed over tp), q / k norms and other replicated parameters inside a parallel region still hold parts;
    losses and gradient norms equal the single-rank run."""
    a, b = str(tmp_path / "one.pt"), str(tmp_path / "tp.pt")
    run_distributed(_run, 1, [], a, 128, timeout=400)
    run_distributed(_run, 2, ["--parallelism.tensor_parallel_degree", "2", "--parallelism.no-enable_sequence_parallel"],
                    b, 128, timeout=400)
    ra, rb = torch.load(a), torch.load(b)
    assert torch.allclose(ra, rb, atol=2e-4), (ra, rb)


def test_async_tensor_parallel_flag_selects_the_fused_gemms():
    """``compile.enable_async_tensor_parallel`` (the reference's switch) maps to the GEMM kernels with the collective
    inside; without sequence parallelism it is refused."""
    from torchtitan_b200.config import ConfigManager

    base = ["--module", "llama3", "--config", "llama3_debugmodel", "--parallelism.tensor_parallel_degree", "2",
            "--compile.enable_async_tensor_parallel"]
    cfg = ConfigManager().parse_args(base)
    cfg.validate()
    assert cfg.parallelism.tp_comm == "nvlink"
    with pytest.raises(ValueError, match="sequence parallelism"):
        ConfigManager().parse_args(base + ["--parallelism.no-enable_sequence_parallel"]).validate()
