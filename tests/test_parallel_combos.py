"""Combinations of parallelisms on CPU / gloo: HSDP (replicate x shard), and pipeline stages whose
parameters use the sharded layout.  Reference cases: tests/integration_tests/features.py (ddp / hsdp / pp+fsdp)."""

import pytest
import torch

from tests.dist_utils import run_distributed


def _run(rank, world, extra, out_path, global_tokens):
    from torchtitan_b200.config import ConfigManager

    args = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "3",
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
