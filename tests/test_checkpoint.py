"""DCP checkpoints: chunk geometry, save/load round trip, resume equivalence, resharding 2 -> 1 ranks,
Hugging Face export/import, retention policy."""

import os
import shutil

import pytest
import torch

from tests.dist_utils import run_distributed
from torchtitan_b200.components.checkpoint import flat_interval_to_boxes


def test_flat_interval_to_boxes_covers_interval_exactly():
    shape = (5, 4, 3)
    total = 60
    for start, length in [(0, 60), (7, 30), (13, 1), (11, 25), (59, 1), (12, 24)]:
        ref = torch.zeros(total)
        ref[start:start + length] = 1
        got = torch.zeros(shape)
        n = 0
        for offs, sizes, foff in flat_interval_to_boxes(shape, start, length):
            view = got
            for d, (o, s) in enumerate(zip(offs, sizes)):
                view = view.narrow(d, o, s)
            view += 1
            n += view.numel()
        assert n == length
        assert torch.equal(got.reshape(-1), ref)


def _args(folder, steps, extra=()):
    return ["--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", str(steps),
            "--training.num_tokens_per_microbatch_per_dp_rank", "64", "--training.max_context_length", "64",
            "--training.mixed_precision_param", "float32", "--debug.seed", "0", "--dump_folder", folder,
            "--debug.no-enable_structured_logging", "--metrics.log_freq", "1", "--checkpoint.enable",
            "--checkpoint.interval", "2", "--checkpoint.no-last_save_model_only", "--lr_scheduler.warmup_steps", "2",
            "--lr_scheduler.total_steps", "6",
            *extra]


def _train(rank, world, folder, steps, out_path, extra=()):
    from torchtitan_b200.config import ConfigManager

    cfg = ConfigManager().parse_args(_args(folder, steps, extra))
    t = cfg.build()
    losses = []
    orig = t.metrics_processor.log

    def log(step, avg, mx, gn, extra_metrics=None):
        losses.append((step, avg))
        return orig(step, avg, mx, gn, extra_metrics=extra_metrics)

    t.metrics_processor.log = log
    t.train()
    if rank == 0:
        torch.save(losses, out_path)
    t.close()


def test_resume_reproduces_uninterrupted_run(tmp_path):
    full, part, resumed = (str(tmp_path / n) for n in ("full.pt", "part.pt", "res.pt"))
    run_distributed(_train, 1, str(tmp_path / "a"), 6, full)
    run_distributed(_train, 1, str(tmp_path / "b"), 4, part)
    assert os.path.exists(tmp_path / "b" / "checkpoint" / "step-4" / ".metadata")
    run_distributed(_train, 1, str(tmp_path / "b"), 6, resumed)
    a, c = dict(torch.load(full)), dict(torch.load(resumed))
    assert sorted(c) == [5, 6]
    for s in (5, 6):
        assert abs(a[s] - c[s]) < 1e-5, (s, a[s], c[s])


def test_two_rank_checkpoint_loads_on_one_rank(tmp_path):
    """Save under FSDP=2, resume model+optimizer under 1 rank: the next losses are finite and the
    parameters equal what rank 0 of the 2-rank job held."""
    two, one = str(tmp_path / "two.pt"), str(tmp_path / "one.pt")
    run_distributed(_train, 2, str(tmp_path / "c"), 2, two)
    # dataloader state is per dp degree: exclude it when the layout changes
    run_distributed(_train, 1, str(tmp_path / "c"), 3, one, ("--checkpoint.exclude_from_loading", "dataloader"))
    losses = dict(torch.load(one))
    assert list(losses) == [3] and losses[3] == losses[3]


def _export(rank, world, folder, hf):
    from torchtitan_b200.config import ConfigManager

    extra = ["--checkpoint.last_save_model_only", "--checkpoint.export_dtype", "bfloat16"]
    if hf:
        extra.append("--checkpoint.last_save_in_hf")
    args = [a for a in _args(folder, 2, extra) if a != "--checkpoint.no-last_save_model_only"]
    t = ConfigManager().parse_args(args).build()
    t.train()
    t.close()


def test_hf_export_and_reimport(tmp_path):
    from safetensors.torch import load_file

    folder = str(tmp_path / "d")
    run_distributed(_export, 1, folder, True)
    path = os.path.join(folder, "checkpoint", "step-2")
    sd = load_file(os.path.join(path, "model.safetensors"))
    assert "model.layers.0.self_attn.q_proj.weight" in sd and sd["lm_head.weight"].dtype == torch.bfloat16
    assert sd["model.layers.0.mlp.gate_proj.weight"].shape == (768, 256)

    # import: a fresh model initialised from the HF folder has the exported weights
    from torchtitan_b200.config import ConfigManager

    cfg = ConfigManager().parse_args(_args(str(tmp_path / "e"), 1, ["--checkpoint.initial_load_path", path,
                                                                      "--checkpoint.initial_load_in_hf"]))
    t = cfg.build()
    assert t.checkpointer.load()
    w = t.model.layers["0"].feed_forward.w13.weight[:768]
    assert torch.allclose(w.bfloat16().float(), sd["model.layers.0.mlp.gate_proj.weight"].float(), atol=1e-6)
    t.close()


def test_adapter_qk_permutation_round_trip():
    from torchtitan_b200.models.state_dict_adapter import halves_to_pairs, pairs_to_halves

    w = torch.randn(4 * 8, 5)
    assert torch.equal(halves_to_pairs(pairs_to_halves(w, 4), 4), w)
    # pairs (0,1),(2,3).. -> halves: first half holds even rows
    one = torch.arange(8.0)[:, None]
    assert pairs_to_halves(one, 1).flatten().tolist() == [0, 2, 4, 6, 1, 3, 5, 7]


@pytest.mark.parametrize("module,flavor,seq", [
    ("llama3", "debugmodel_gqa", 48), ("qwen3", "debugmodel", 48), ("qwen3", "debugmodel_moe_tiny", 48),
    ("deepseek_v3", "debugmodel_v3routing", 48), ("gpt_oss", "debugmodel", 96), ("qwen3_5", "debugmodel", 100),
    ("qwen3_5", "debugmodel_moe", 80)])
def test_logits_match_transformers_on_converted_weights(module, flavor, seq):
    """A freshly initialised Hugging Face model and the native model that received its weights through the family's
    state-dict adapter give the same next-token distributions: mean KL below 1e-6.  Covers the RoPE conventions and
    their Llama / YaRN scalings, fused q/k/v and gate/up splits, grouped queries, q/k norms, tied embeddings, top-k
    routers (softmax, and sigmoid with groups, bias and scaling), shared experts, multi-head latent attention, and
    GPT-OSS's sinks, alternating sliding window (sequence longer than the window), biases and clamped SwiGLU, and
    Qwen3.5's Gated DeltaNet layers (fused projections and convolution, chunked delta rule across chunk boundaries,
    gated norm), gated partial-rotary attention, offset-gain norms and gated shared expert.  Norm gains, biases and
    the other 1-D parameters are perturbed so that they matter."""
    pytest.importorskip("transformers")
    from torchtitan_b200.scripts.numerical_tests import main

    res = main(["--module", module, "--flavor", flavor, "--random", "--perturb", "0.1", "--seq-len", str(seq),
                "--num-seqs", "2", "--grads"])
    assert abs(res["kl_mean"]) < 1e-6 and res["max_abs_logit_diff"] < 1e-4, res
    # the backward of the native operators against transformers' autograd, parameter by parameter
    assert res["grad_tensors_compared"] >= 20 and res["max_rel_grad_diff"] < 2e-3, res


def test_qwen3_5_adapter_round_trip():
    """Native -> Hugging Face -> native is the identity for the Qwen3.5 layouts (fused DeltaNet projections and
    convolution, query / gate interleaving, fused expert tensors), with either decoder prefix."""
    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.models.common.module import iter_checkpoint_slices

    for flavor in ("debugmodel", "debugmodel_moe"):
        spec = get_model_spec("qwen3_5", flavor)
        model = spec.model.build()
        model.init_states(seed=3)
        fused = dict(iter_checkpoint_slices(model))
        native = {}
        for k, p in model.named_parameters():
            if k in fused:
                for name, a, b in fused[k]:
                    native[name] = p.detach()[a:b].clone()
            else:
                native[k] = p.detach().clone()
        ad = spec.state_dict_adapter(spec.model, None)
        for prefix in ("model.language_model.", "model."):
            ad.hf_prefix = prefix
            hf = ad.to_hf(dict(native))
            assert all(k.startswith(prefix) or k == "lm_head.weight" for k in hf), list(hf)[:3]
            assert any(k.endswith("linear_attn.in_proj_qkv.weight") for k in hf)
            back = ad.from_hf(hf)
            assert set(back) == set(native), set(back) ^ set(native)
            for k in native:
                assert torch.equal(back[k], native[k]), k


def test_torch_save_storage_resumes_and_reshards(tmp_path):
    """``checkpoint.storage = torch_save`` (one file per rank with global chunk offsets): a 2-rank job resumes exactly
    from its own files, and its checkpoint loads on 1 rank (model and optimizer re-laid-out by box overlap) where the
    next loss equals the one of loading the same step from DCP files."""
    ts = ("--checkpoint.storage", "torch_save")
    full, resumed, one_ts, one_dcp = (str(tmp_path / n) for n in ("full.pt", "res.pt", "one_ts.pt", "one_dcp.pt"))
    run_distributed(_train, 2, str(tmp_path / "a"), 4, full, ts)
    run_distributed(_train, 2, str(tmp_path / "b"), 2, str(tmp_path / "part.pt"), ts)
    assert os.path.exists(tmp_path / "b" / "checkpoint" / "step-2" / "rank-1.pt")
    run_distributed(_train, 2, str(tmp_path / "b"), 4, resumed, ts)
    a, c = dict(torch.load(full)), dict(torch.load(resumed))
    assert sorted(c) == [3, 4]
    for s in (3, 4):
        assert abs(a[s] - c[s]) < 1e-5, (s, a[s], c[s])
    # the same two training steps written by both engines, then loaded on one rank
    run_distributed(_train, 2, str(tmp_path / "d"), 2, str(tmp_path / "y.pt"))
    skip = ("--checkpoint.exclude_from_loading", "dataloader")
    shutil.rmtree(tmp_path / "b" / "checkpoint" / "step-4")            # folder b still holds the torch.save step 2
    run_distributed(_train, 1, str(tmp_path / "b"), 3, one_ts, ts + skip)
    run_distributed(_train, 1, str(tmp_path / "d"), 3, one_dcp, skip)
    x, y = dict(torch.load(one_ts)), dict(torch.load(one_dcp))
    assert list(x) == [3] and abs(x[3] - y[3]) < 1e-6, (x, y)


def test_filesystem_helpers_local_and_fsspec(tmp_path):
    from torchtitan_b200.utils import filesystem as fsys

    for root in (str(tmp_path / "loc"), "memory://fs_helpers_test"):
        assert fsys.is_remote(root) == root.startswith("memory://")
        assert fsys.listdir(root) == [] and not fsys.exists(root)
        d = fsys.join(root, "step-3")
        fsys.makedirs(d)
        with fsys.open_file(fsys.join(d, ".metadata"), "w") as f:
            f.write("x")
        assert fsys.isdir(d) and fsys.isfile(fsys.join(d, ".metadata")) and fsys.listdir(root) == ["step-3"]
        assert fsys.listdir(d) == [".metadata"]
        fsys.rmtree(d)
        assert not fsys.exists(d)
    assert not fsys.is_remote("file:///tmp/x") and not fsys.is_remote("C:/x") and fsys.is_remote("s3://b/k")
    assert fsys.join("s3://b/run/", "/checkpoint/", "step-1") == "s3://b/run/checkpoint/step-1"


def _train_remote(rank, world, folder, steps, out_path):
    _train(rank, world, folder, steps, out_path, ("--checkpoint.folder", "memory://ckpt_remote_test", "--checkpoint.keep_latest_k", "2"))
    from torchtitan_b200.utils import filesystem as fsys

    if rank == 0:
        torch.save(fsys.listdir("memory://ckpt_remote_test"), out_path + ".ls")


def test_checkpoints_on_an_fsspec_uri(tmp_path):
    """``checkpoint.folder`` as an fsspec URI (the in-process ``memory://`` filesystem here): DCP writes through its
    fsspec storage, step discovery and the retention policy work on the URI."""
    out = str(tmp_path / "o.pt")
    run_distributed(_train_remote, 1, str(tmp_path / "r"), 6, out)
    kept = torch.load(out + ".ls")
    assert "step-6" in kept and "step-2" not in kept and len([k for k in kept if k.startswith("step-")]) <= 3, kept
    assert not os.path.exists(tmp_path / "r" / "checkpoint")
