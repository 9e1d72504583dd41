"""Pipeline parallel: stage assignment rules and 2-stage training parity with a single process."""

import pytest
import torch

from tests.dist_utils import run_distributed
from torchtitan_b200.parallel.pipeline import stage_ids_for_rank, stage_layer_assignment


def test_stage_assignment_rules():
    a = stage_layer_assignment(6, 2)
    assert a == [(True, [0, 1, 2], False), (False, [3, 4, 5], True)]
    a = stage_layer_assignment(8, 4)
    assert [len(x[1]) for x in a] == [2, 3, 2, 1] or sum(len(x[1]) for x in a) == 8
    assert sum(len(x[1]) for x in a) == 8 and a[0][0] and a[-1][2]
    assert stage_ids_for_rank(1, 2, 4) == [1, 3]
    assert stage_ids_for_rank(0, 2, 4, "v") == [0, 3]


def _run(rank, world, schedule, out_path):
    from torchtitan_b200.config import ConfigManager

    args = ["--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "3",
            "--training.num_tokens_per_microbatch_per_dp_rank", "64", "--training.max_context_length", "64",
            "--training.mixed_precision_param", "float32", "--debug.seed", "0", "--dump_folder", out_path + "_d",
            "--debug.no-enable_structured_logging", "--metrics.log_freq", "1"]
    if world > 1:
        args += ["--parallelism.pipeline_parallel_degree", "2", "--parallelism.pipeline_parallel_schedule", schedule,
                 "--parallelism.num_pp_microbatches", "2"]
    else:
        args += ["--training.num_tokens_per_train_step", "128"]
    cfg = ConfigManager().parse_args(args)
    t = cfg.build()
    losses = []
    orig = t.metrics_processor.log

    def log(step, avg, mx, gn, extra_metrics=None):
        losses.append(avg)
        return orig(step, avg, mx, gn, extra_metrics=extra_metrics)

    t.metrics_processor.log = log
    t.train()
    if rank == 0:
        torch.save(torch.tensor(losses), out_path)
    t.close()


@pytest.mark.parametrize("schedule", ["1F1B", "Interleaved1F1B"])
def test_pp_matches_single_process(tmp_path, schedule):
    single, piped = str(tmp_path / "s.pt"), str(tmp_path / "p.pt")
    run_distributed(_run, 1, "none", single)
    run_distributed(_run, 2, schedule, piped, timeout=400)
    a, b = torch.load(single), torch.load(piped)
    assert torch.allclose(a, b, atol=2e-4), (a, b)
