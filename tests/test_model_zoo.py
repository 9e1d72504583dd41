"""Every registered model family builds, trains two steps on CPU through the trainer, and its
parameter accounting and checkpoint-name adapter agree with the module tree."""

import pytest
import torch

from torchtitan_b200.config import ConfigManager
from torchtitan_b200.models import get_model_spec
from torchtitan_b200.models.utils import count_params_and_flops

FAMILIES = [
    ("llama3", "llama3_debugmodel", "debugmodel"),
    ("qwen3", "qwen3_debugmodel", "debugmodel"),
    ("qwen3", "qwen3_moe_tiny", "debugmodel_moe_tiny"),
    ("deepseek_v3", "deepseek_v3_debugmodel", "debugmodel"),
    ("deepseek_v3", "deepseek_v3_debugmodel_mtp", "debugmodel_mtp"),
    ("gpt_oss", "gpt_oss_debugmodel", "debugmodel"),
    ("muse_glimmer", "muse_glimmer_debugmodel", "debugmodel"),
    ("kimi_k2_7", "kimi_debugmodel", "debugmodel"),
    ("kimi_k2_7", "kimi_debugmodel_muon", "debugmodel"),
    ("qwen3_5", "qwen3_5_debugmodel", "debugmodel"),
    ("qwen3_5", "qwen3_5_moe_debug", "debugmodel_moe"),
    ("qwen3_5", "qwen3_5_debugmodel_vl", "debugmodel_vl"),
    ("kimi_k2_7", "kimi_debugmodel_vl", "debugmodel_vl"),
    ("muse_glimmer", "muse_glimmer_debugmodel_mm", "debugmodel_mm"),
]


@pytest.mark.parametrize("module,config,flavor", FAMILIES)
def test_family_trains_on_cpu(module, config, flavor, tmp_path):
    cfg = ConfigManager().parse_args([
        "--module", module, "--config", config, "--training.steps", "2",
        "--training.num_tokens_per_microbatch_per_dp_rank", "128", "--training.max_context_length", "64",
        "--training.mixed_precision_param", "float32", "--debug.seed", "0", "--dump_folder", str(tmp_path),
        "--debug.no-enable_structured_logging", "--checkpoint.no-enable",
    ])
    trainer = cfg.build()
    trainer.train()
    loss = float(trainer._last_loss)
    assert loss == loss and 3.0 < loss < 12.0, loss
    trainer.close()


@pytest.mark.parametrize("module,flavor", [(m, f) for m, _, f in FAMILIES])
def test_param_count_matches_module_tree(module, flavor):
    spec = get_model_spec(module, flavor)
    with torch.device("meta"):
        model = spec.model.build()
    n_module = sum(p.numel() for n, p in model.named_parameters())
    if spec.model.enable_weight_tying:
        n_module = sum(p.numel() for p in {id(p): p for p in model.parameters()}.values())
    n_cfg, flops = count_params_and_flops(spec.model, model, 2048)
    assert n_cfg == n_module, (n_cfg, n_module)
    assert flops > 0


def test_gated_delta_rule_chunked_equals_recurrent():
    from torchtitan_b200.models.qwen3_5.gdn import causal_conv_silu, chunk_gated_delta_rule, recurrent_gated_delta_rule

    torch.manual_seed(0)
    T, H, dk, dv = 150, 3, 16, 24
    q, k, v = torch.randn(T, H, dk), torch.randn(T, H, dk), torch.randn(T, H, dv)
    g, beta = -torch.rand(T, H) * 0.5, torch.rand(T, H)
    g[70] = -1e3  # a document boundary: the state restarts
    a, b = recurrent_gated_delta_rule(q, k, v, g, beta), chunk_gated_delta_rule(q, k, v, g, beta, chunk=32)
    assert torch.allclose(a, b, atol=1e-4)
    assert torch.allclose(a[70:], recurrent_gated_delta_rule(q[70:], k[70:], v[70:], g[70:], beta[70:]), atol=1e-5)
    # the convolution does not reach across a document start
    x, w = torch.randn(20, 6), torch.randn(6, 4)
    pos = torch.cat([torch.arange(12), torch.arange(8)])
    y = causal_conv_silu(x, w, pos)
    assert torch.allclose(y[12:], causal_conv_silu(x[12:], w, None), atol=1e-6)


@pytest.mark.parametrize("module,flavor", [("deepseek_v3", "debugmodel"), ("gpt_oss", "debugmodel"), ("qwen3", "debugmodel_moe")])
def test_hf_adapter_round_trip(module, flavor):
    from torchtitan_b200.models.common.module import iter_checkpoint_slices

    spec = get_model_spec(module, flavor)
    model = spec.model.build()
    model.init_states(seed=0)
    fused = dict(iter_checkpoint_slices(model))
    native = {}
    for k, v in list(model.named_parameters()) + [(k, b) for k, b in model.named_buffers() if k.endswith("expert_bias_E")]:
        if k in fused:  # checkpoints hold the un-fused pieces (wq / wk / wv, w1 / w3)
            for name, a, b in fused[k]:
                native[name] = v.detach()[a:b]
        else:
            native[k] = v.detach()
    adapter = spec.state_dict_adapter(spec.model, None)
    hf = adapter.to_hf(native)
    back = adapter.from_hf(hf)
    for k, v in native.items():
        if k.endswith("expert_bias_E") and k not in back:
            continue
        assert k in back, k
        assert torch.equal(back[k], v), k


def test_flux_flow_matching_trains():
    from torchtitan_b200.models.flux.config_registry import flux_debugmodel

    cfg = flux_debugmodel()
    cfg.steps = 12
    cfg.lr = 2e-3
    tr = cfg.build()
    losses = []
    for _ in range(cfg.steps):
        tr.gen.manual_seed(123)          # the same batch, noise and timesteps every step: the loss must fall
        losses.append(tr.train_step())
    assert all(l == l for l in losses)
    assert abs(losses[0] - 2.0) < 0.5    # the model starts as the zero map: E|noise - x0|^2 = 2
    assert losses[-1] < 0.8 * losses[0]


def test_mtp_roll_respects_documents():
    from torchtitan_b200.models.deepseek_v3.mtp import roll_mtp_sequence

    seq = torch.tensor([10, 11, 12, 20, 21])
    pos = torch.tensor([0, 1, 2, 0, 1])
    out, valid = roll_mtp_sequence(seq, shift=1, fill_value=-1, positions=pos, return_valid_mask=True)
    assert out.tolist() == [11, 12, -1, 21, -1] and valid.tolist() == [True, True, False, True, False]
    assert roll_mtp_sequence(seq, shift=2, fill_value=-1, positions=pos).tolist() == [12, -1, -1, -1, -1]
    assert roll_mtp_sequence(seq, shift=2, fill_value=0).tolist() == [12, 20, 21, 0, 0]


def test_mtp_loss_is_main_plus_scaled_depth_mean():
    """The trainer's MTP loss equals the formula evaluated on materialised logits."""
    from torchtitan_b200.components.loss import IGNORE_INDEX
    from torchtitan_b200.models.deepseek_v3.mtp import MTPDecoder, roll_mtp_sequence

    spec = get_model_spec("deepseek_v3", "debugmodel_mtp")
    assert isinstance(spec.model, MTPDecoder.Config) and len(spec.model.mtp_layers) == 2
    model = spec.model.build()
    model.init_states(seed=3)
    T = 48
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 2048, (T + 1,), generator=g)
    tok, lab = ids[:-1], ids[1:].clone()
    pos = torch.cat([torch.arange(30), torch.arange(18)])
    logits = model(tok, pos)
    assert isinstance(logits, list) and len(logits) == 3
    ce = lambda lg, lb: torch.nn.functional.cross_entropy(lg.float(), lb, ignore_index=IGNORE_INDEX, reduction="sum")
    want = ce(logits[0], lab) + 0.3 / 2 * sum(
        ce(logits[k], roll_mtp_sequence(lab, shift=k, fill_value=IGNORE_INDEX, positions=pos)) for k in (1, 2))
    want = want / T

    from torchtitan_b200.components.loss import LinearCrossEntropyLoss
    from torchtitan_b200.models.deepseek_v3.mtp import MTPLoss

    inner = LinearCrossEntropyLoss()
    inner.set_lm_head(model.lm_head)
    loss_fn = MTPLoss(inner, mtp_scale=0.3)
    hidden = model(tok, pos, return_hidden=True)
    got = loss_fn(hidden, lab, torch.tensor(float(T)), positions=pos)
    assert torch.allclose(got, want, rtol=1e-4), (got, want)
    got.backward()
    assert all(p.grad is not None or getattr(p, "main_grad", None) is not None
               for n, p in model.named_parameters() if "mtp_layers" in n and "moe" not in n)


def test_flux_autoencoder_and_sampling(tmp_path):
    from torchtitan_b200.models.flux.autoencoder import AutoEncoder
    from torchtitan_b200.models.flux.config_registry import flux_debugmodel
    from torchtitan_b200.models.flux.sampling import get_schedule, unpack_latents
    from torchtitan_b200.models.flux.trainer import pack_latents

    ae_cfg = AutoEncoder.Config(resolution=32, ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1, z_channels=16)
    ae = ae_cfg.build()
    ae.init_states(seed=0)
    names = set(dict(ae.named_parameters()))
    for n in ("encoder.down.0.block.0.conv1.weight", "encoder.down.0.downsample.conv.weight", "encoder.mid.attn_1.q.weight",
              "decoder.up.3.upsample.conv.weight", "decoder.up.0.block.1.norm2.weight", "decoder.conv_out.bias"):
        assert n in names, n
    assert "encoder.down.3.downsample.conv.weight" not in names and "decoder.up.0.upsample.conv.weight" not in names
    x = torch.rand(2, 3, 32, 32) * 2 - 1
    z = ae.encode(x)
    assert z.shape == (2, 16, 4, 4) and ae.decode(z).shape == x.shape and ae.downsample_factor == 8
    lat = torch.randn(2, 16, 6, 4)
    assert torch.equal(unpack_latents(pack_latents(lat), 6, 4), lat)
    ts = get_schedule(8, 64)
    assert ts[0] == 1.0 and ts[-1] == 0.0 and all(a > b for a, b in zip(ts, ts[1:]))
    assert get_schedule(8, 4096)[4] > get_schedule(8, 256)[4] > get_schedule(8, 256, shift=False)[4] - 1e-9

    cfg = flux_debugmodel()
    cfg.steps, cfg.img_size, cfg.autoencoder = 2, 32, ae_cfg
    trainer = cfg.build()
    trainer.train()
    v = trainer.validate()
    assert v == v and v > 0
    out = str(tmp_path / "sample.png")
    img = trainer.generate(torch.randint(0, 1024, (1, cfg.txt_len)), steps=2, guidance_scale=2.0, path=out)
    assert img.shape == (1, 3, 32, 32) and torch.isfinite(img).all()
    import os

    assert os.path.exists(out) or os.path.exists(out[:-4] + ".ppm")


def test_every_registered_config_builds_its_model_on_meta():
    """Each config-registry function returns a config whose model flavor exists and builds on the
    meta device with a parameter count that matches its accounting."""
    import importlib
    import inspect

    from torchtitan_b200.models.spec import SUPPORTED_MODELS

    n = 0
    for fam in SUPPORTED_MODELS:
        if fam == "flux":
            continue
        reg = importlib.import_module(f"torchtitan_b200.models.{fam}.config_registry")
        for name, fn in inspect.getmembers(reg, inspect.isfunction):
            if name.startswith("_") or fn.__module__ != reg.__name__ or inspect.signature(fn).parameters:
                continue
            cfg = fn()
            spec = get_model_spec(cfg.model.name, cfg.model.flavor)
            if "debug" in cfg.model.flavor:
                from torchtitan_b200.components.quantization import apply_converters

                apply_converters(spec.model, cfg.model.converters)
                with torch.device("meta"):
                    model = spec.model.build()
                assert sum(p.numel() for p in model.parameters()) > 0
            else:
                total, flops = count_params_and_flops(spec.model, None, 4096)
                assert total > 1e8 and flops > 0, (fam, name, total)
            n += 1
    assert n >= 50
