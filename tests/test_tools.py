"""Scripts and tools: HF conversion round trip, loss comparison, activation tracing."""

import os

import torch

from torchtitan_b200.models import get_model_spec


def test_convert_hf_round_trip(tmp_path):
    import torch.distributed.checkpoint as dcp

    from torchtitan_b200.scripts import convert_hf

    spec = get_model_spec("llama3", "debugmodel")
    tmpl = convert_hf._native_template(spec)
    g = torch.Generator().manual_seed(0)
    state = {f"model.{k}": torch.randn(shape, generator=g) for k, (_, _, shape) in tmpl.items()}
    ck = str(tmp_path / "step-1")
    dcp.save(state, checkpoint_id=ck, no_dist=True)
    convert_hf.main(["to_hf", "--module", "llama3", "--flavor", "debugmodel", "--checkpoint", ck,
                     "--out", str(tmp_path / "hf"), "--dtype", "float32"])
    assert os.path.exists(tmp_path / "hf" / "model.safetensors.index.json")
    convert_hf.main(["from_hf", "--module", "llama3", "--flavor", "debugmodel", "--hf-dir", str(tmp_path / "hf"),
                     "--out", str(tmp_path / "back"), "--dtype", "float32"])
    back = {k: torch.empty_like(v) for k, v in state.items()}
    dcp.load(back, checkpoint_id=str(tmp_path / "back"), no_dist=True)
    for k in state:
        assert torch.equal(state[k], back[k]), k


def test_loss_compare_detects_equal_and_different(tmp_path):
    from torchtitan_b200.scripts import loss_compare

    base = ("--module llama3 --config llama3_debugmodel --training.num_tokens_per_microbatch_per_dp_rank 128 "
            "--training.max_context_length 64 --training.mixed_precision_param float32")
    golden = str(tmp_path / "golden.json")
    assert loss_compare.main(["--baseline", base, "--test", base, "--steps", "3", "--assert-equal",
                              "--export", golden]) == 0
    assert loss_compare.main(["--import", golden, "--test", base + " --optimizer.lr 1e-2", "--steps", "3",
                              "--assert-equal"]) == 1


def test_activation_tracer_finds_first_divergence():
    from torchtitan_b200.tools.numerics import ActivationTracer, compare_traces

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.ReLU(), torch.nn.Linear(8, 4))
    x = torch.randn(5, 8)
    with ActivationTracer(net, grads=True) as a:
        net(x).sum().backward()
    with ActivationTracer(net, grads=True) as b:
        net(x).sum().backward()
    assert "no statistic differs" in compare_traces(a, b)
    with torch.no_grad():
        net[2].weight.mul_(3.0)
    with ActivationTracer(net) as c:
        net(x)
    rep = compare_traces([r for r in a.records if r["kind"] == "out"], c)
    assert "first divergence" in rep and ": 2 (" in rep


def test_download_asset_selection():
    from torchtitan_b200.scripts.download_hf_assets import select_files

    files = ["config.json", "tokenizer.json", "model-00001-of-00002.safetensors", "model.safetensors.index.json",
             "original/consolidated.pth", "README.md"]
    assert select_files(files, ["tokenizer", "config"], []) == ["config.json", "tokenizer.json"]
    assert select_files(files, ["index", "safetensors"], ["original/*"]) == [
        "model-00001-of-00002.safetensors", "model.safetensors.index.json", "original/consolidated.pth"]


def test_checkpoint_compat_script_same_revision(tmp_path):
    """Saving and resuming with the working tree itself must reproduce the uninterrupted run."""
    from torchtitan_b200.scripts import checkpoint_compat_test as cc

    args = ("--module llama3 --config llama3_debugmodel --training.num_tokens_per_microbatch_per_dp_rank 128 "
            "--training.max_context_length 64 --training.mixed_precision_param float32")
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a = cc.run(root, args, str(tmp_path / "r"), 2, 1)
    resumed = cc.run(root, args, str(tmp_path / "r"), 4, 1)
    straight = cc.run(root, args, str(tmp_path / "s"), 4, 1)
    assert [s for s, _ in a] == [1, 2] and [s for s, _ in resumed] == [3, 4]
    assert resumed == straight[2:]


def test_operator_tracer_and_html_report(tmp_path):
    import torch

    from torchtitan_b200.tools.numerics import OperatorTracer, html_report

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.GELU(), torch.nn.Linear(16, 4))
    x = torch.randn(5, 8)
    with OperatorTracer(net) as a:
        net(x).sum().backward()
    with torch.no_grad():
        net[2].weight.mul_(1.5)
    with OperatorTracer(net) as b:
        net(x).sum().backward()
    assert any("addmm" in r["name"] or "mm" in r["name"] for r in a.records)
    assert any(r["name"].startswith("2::") for r in a.records)          # tagged with the executing module
    out = tmp_path / "report.html"
    n = html_report(a, b, str(out))
    text = out.read_text()
    assert n > 0 and "class='diff'" in text and "class='same'" in text


def test_memory_plan_of_large_registry_configs():
    """Meta-device memory plans: Llama-3 405B and Qwen3 235B-A22B fit a 180 GB GPU only with sharded parameters;
    the 8B headline at 8 GPUs keeps at most its shards plus four unit-sized slots in the sharded layout."""
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.tools.memory_plan import plan_memory

    def cfg(module, name, *extra):
        return ConfigManager().parse_args(["--module", module, "--config", name, *extra])

    c = cfg("llama3", "llama3_405b", "--parallelism.tensor_parallel_degree", "8", "--parallelism.pipeline_parallel_degree", "1",
            "--parallelism.fsdp_reshard_after_forward", "default")
    big = plan_memory(c, world=512)
    assert big.layout == "sharded parameters" and big.fits(), str(big)
    c.parallelism.fsdp_reshard_after_forward = "never"
    assert not plan_memory(c, world=512).fits()
    moe = plan_memory(cfg("qwen3", "qwen3_235b_a22b", "--parallelism.fsdp_reshard_after_forward", "always",
                          "--parallelism.expert_parallel_degree", "8", "--parallelism.pipeline_parallel_degree", "1",
                          "--parallelism.tensor_parallel_degree", "1"), world=128)
    assert moe.fits(), str(moe)
    small = cfg("llama3", "llama3_8b", "--parallelism.fsdp_reshard_after_forward", "always")
    p8 = plan_memory(small, world=8)
    full_bf16 = 8.03e9 * 2 / (1 << 30)
    assert p8.params_gib <= full_bf16 / 8 + 2 * p8.largest_unit_gib + 0.1, str(p8)
    resident = plan_memory(cfg("llama3", "llama3_8b", "--parallelism.fsdp_reshard_after_forward", "never"), world=8)
    assert resident.params_gib > 0.95 * full_bf16
