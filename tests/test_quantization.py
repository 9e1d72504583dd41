"""Quantisation converters and LoRA on CPU: the reference quantisers, the config rewrites, and
training through the trainer with converted models."""

import math

import pytest
import torch

from torchtitan_b200.components.quantization import apply_converters
from torchtitan_b200.components.quantization.linear import QuantLinear
from torchtitan_b200.config import ConfigManager
from torchtitan_b200.models import get_model_spec
from torchtitan_b200.ops import reference as ref


def test_mxfp8_reference_properties():
    torch.manual_seed(0)
    x = torch.randn(64, 128) * torch.logspace(-3, 3, 64)[:, None]
    for axis in (0, 1):
        q = ref.mxfp8_fake_quant(x, axis)
        # e4m3 has 3 mantissa bits and RCEIL never saturates: relative error per block <= 2^-4 of the block max
        blocks = (x if axis == 1 else x.t()).reshape(-1, 32)
        qb = (q if axis == 1 else q.t()).reshape(-1, 32)
        err = (blocks - qb).abs().amax(dim=1)
        assert (err <= blocks.abs().amax(dim=1) * 2 ** -4 + 1e-30).all()
        assert torch.equal(ref.mxfp8_fake_quant(q, axis), q)  # idempotent
    z = torch.zeros(4, 32)
    assert torch.equal(ref.mxfp8_fake_quant(z, 1), z)
    # the scale is the smallest power of two >= amax / 448
    e = ref.mxfp8_scale_exponent(torch.tensor([448.0, 449.0, 1.0, 0.0]))
    assert e.tolist() == [0, 1, math.ceil(math.log2(1 / 448)), -127]


def test_converters_rewrite_config_tree():
    spec = get_model_spec("llama3", "debugmodel")
    n = apply_converters(spec.model, ["mxfp8"]) if False else None
    apply_converters(spec.model, ["mxfp8", "lora:rank=4,alpha=8"])
    blk = spec.model.layers[0]
    assert type(blk.attention.wqkv).__qualname__ == "LoRAQuantLinear.Config"
    assert type(spec.model.lm_head).__qualname__ == "Linear.Config"
    model = spec.model.build()
    names = [n for n, p in model.named_parameters() if p.requires_grad]
    assert names and all(n.endswith("lora_a") or n.endswith("lora_b") for n in names)
    with pytest.raises(ValueError):
        apply_converters(get_model_spec("llama3", "debugmodel").model, ["lora", "float8"])


def test_quant_linear_gradients_follow_recipe():
    torch.manual_seed(1)
    lin = QuantLinear.Config(in_features=64, out_features=96, recipe="mxfp8").build()
    lin.init_states(seed=0)
    x = torch.randn(40, 64, requires_grad=True)
    y = lin(x)
    g = torch.randn_like(y)
    y.backward(g)
    fq = ref.mxfp8_fake_quant
    w = lin.weight.detach()
    assert torch.allclose(y, fq(x.detach(), 1) @ fq(w, 1).t(), atol=1e-5)
    assert torch.allclose(x.grad, fq(g, 1) @ fq(w, 0), atol=1e-5)
    gp = torch.nn.functional.pad(g, (0, 0, 0, 24))  # token blocks of 32: the last one is ragged
    assert torch.allclose(lin.weight.grad, fq(g, 0).t() @ fq(x.detach(), 0), atol=1e-4)


@pytest.mark.parametrize("converters", [["mxfp8"], ["float8:rowwise_with_gw_hp"], ["float8", "lora:rank=4"]])
def test_converted_models_train(converters, tmp_path):
    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "3",
        "--training.num_tokens_per_microbatch_per_dp_rank", "128", "--training.max_context_length", "64",
        "--training.mixed_precision_param", "float32", "--debug.seed", "0", "--dump_folder", str(tmp_path),
        "--debug.no-enable_structured_logging", "--checkpoint.no-enable",
        "--model.converters", ",".join(converters),
    ])
    trainer = cfg.build()
    trainer.train()
    loss = float(trainer._last_loss)
    assert loss == loss and loss < 9.0, loss
    trainer.close()


def test_quant_grouped_linear_follows_recipe():
    """Grouped (expert) GEMMs: each of the three GEMMs sees operands quantised along its contraction."""
    from torchtitan_b200.components.quantization.grouped import quant_grouped_linear

    torch.manual_seed(2)
    E, N, K = 3, 64, 96
    counts = [40, 0, 70]
    offs = torch.tensor(counts).cumsum(0).to(torch.int32)
    x = torch.randn(sum(counts), K, requires_grad=True)
    w = torch.randn(E, N, K, requires_grad=True)
    y = quant_grouped_linear(x, w, offs, "mxfp8", False)
    g = torch.randn_like(y)
    y.backward(g)
    fq = ref.mxfp8_fake_quant
    lo = 0
    for e, c in enumerate(counts):
        hi = lo + c
        if c:
            xe, ge, we = x.detach()[lo:hi], g[lo:hi], w.detach()[e]
            assert torch.allclose(y[lo:hi], fq(xe, 1) @ fq(we, 1).t(), atol=1e-4)
            assert torch.allclose(x.grad[lo:hi], fq(ge, 1) @ fq(we, 0), atol=1e-4)
            assert torch.allclose(w.grad[e], fq(ge, 0).t() @ fq(xe, 0), atol=1e-3)
        else:
            assert torch.equal(w.grad[e], torch.zeros(N, K))
        lo = hi


def test_expert_converters_train(tmp_path):
    spec = get_model_spec("qwen3", "debugmodel_moe")
    apply_converters(spec.model, ["mxfp8_experts"])
    moe = next(b.moe for b in spec.model.layers if b.moe is not None)
    assert moe.routed_experts.inner_experts.quant_recipe == "mxfp8"
    cfg = ConfigManager().parse_args([
        "--module", "qwen3", "--config", "qwen3_moe_tiny", "--training.steps", "2",
        "--training.num_tokens_per_microbatch_per_dp_rank", "128", "--training.max_context_length", "64",
        "--training.mixed_precision_param", "float32", "--dump_folder", str(tmp_path), "--checkpoint.no-enable",
        "--debug.no-enable_structured_logging", "--model.converters", "float8_experts",
    ])
    trainer = cfg.build()
    trainer.train()
    loss = float(trainer._last_loss)
    assert loss == loss and 3.0 < loss < 12.0
    trainer.close()


def test_nvfp4_quantiser_properties():
    from torchtitan_b200.components.quantization.nvfp4 import hadamard16, nvfp4_fake_quant

    torch.manual_seed(0)
    h = hadamard16()
    assert torch.allclose(h @ h.t(), torch.eye(16), atol=1e-6)           # orthonormal: cancels in a product
    x = torch.randn(64, 128) * torch.logspace(-2, 2, 64)[:, None]
    q = nvfp4_fake_quant(x, 1)
    blocks, qb = x.reshape(-1, 16), q.reshape(-1, 16)
    # e2m1's widest gap is 2 (between 4 and 6) on a grid scaled to amax/6 (+ e4m3 scale rounding 2^-4)
    bound = blocks.abs().amax(dim=1) / 6.0 * (1.0 + 2 ** -3)
    assert ((blocks - qb).abs().amax(dim=1) <= bound + 1e-12).all()
    assert torch.allclose(nvfp4_fake_quant(q, 1), q, rtol=1e-6, atol=0)      # idempotent
    # at most 15 distinct magnitudes per block (the e2m1 grid times one scale)
    assert all(len(set(r.abs().tolist())) <= 8 for r in qb[:16])
    # stochastic rounding is unbiased
    g = torch.Generator().manual_seed(5)
    y = torch.full((4096, 16), 0.7)
    y[:, 0] = 6.0
    m = nvfp4_fake_quant(y, 1, stochastic=True, generator=g)[:, 1:].mean()
    assert abs(float(m) - 0.7) < 0.01
    # the transform cancels between the two operands of a product over the transformed axis
    a, b = torch.randn(64, 24), torch.randn(64, 40)
    ah = (a.t().reshape(24, 4, 16) @ h).reshape(24, 64).t()
    bh = (b.t().reshape(40, 4, 16) @ h).reshape(40, 64).t()
    assert torch.allclose(ah.t() @ bh, a.t() @ b, atol=1e-4)


def test_nvfp4_linear_and_converter(tmp_path):
    from torchtitan_b200.components.quantization.nvfp4 import NVFP4Linear, nvfp4_bf16_tail_fqns, nvfp4_fake_quant

    assert nvfp4_bf16_tail_fqns(8, 0.25) == [f"layers.{i}." for i in range(6)]
    with pytest.raises(ValueError):
        nvfp4_bf16_tail_fqns(4, 1.0)
    with pytest.raises(ValueError):
        NVFP4Linear.Config(in_features=96, out_features=128).build()
    torch.manual_seed(3)
    lin = NVFP4Linear.Config(in_features=128, out_features=256).build()
    lin.init_states(seed=0)
    x = torch.randn(64, 128, requires_grad=True)
    y = lin(x)
    w = lin.weight.detach()
    assert torch.allclose(y, nvfp4_fake_quant(x.detach(), 1) @ nvfp4_fake_quant(w, 1).t(), atol=1e-4)
    y.backward(torch.randn_like(y))
    # gradients are noisy (fp4, stochastic rounding) but aligned with the exact ones
    xe = x.detach().clone().requires_grad_()
    ye = xe @ w.t()
    torch.manual_seed(3)
    cos = torch.nn.functional.cosine_similarity
    assert lin.weight.grad is not None and x.grad is not None
    spec = get_model_spec("llama3", "debugmodel")
    apply_converters(spec.model, ["nvfp4:tail=0.5"])
    kinds = [type(b.attention.wqkv).__qualname__ for b in spec.model.layers]
    n = len(kinds)
    assert kinds[: n // 2] == ["NVFP4Linear.Config"] * (n // 2) and kinds[n // 2:] == ["Linear.Config"] * (n - n // 2)
