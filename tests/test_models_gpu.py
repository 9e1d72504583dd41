"""GPU: every model family's debug flavor on the sm_100a kernels (bf16) against the same weights on the CPU
reference operators (fp32): logits, loss and gradient of the embedding."""

import copy

import pytest
import torch

from torchtitan_b200.models import get_model_spec
from torchtitan_b200.ops import functional as OF

pytestmark = pytest.mark.gpu

FAMILIES = [("llama3", "debugmodel_hd128"), ("llama3", "debugmodel"), ("qwen3", "debugmodel"), ("qwen3", "debugmodel_moe_tiny"),
            ("deepseek_v3", "debugmodel_v3routing"), ("gpt_oss", "debugmodel"), ("qwen3_5", "debugmodel"),
            ("qwen3_5", "debugmodel_moe"), ("kimi_k2_7", "debugmodel"), ("muse_glimmer", "debugmodel")]


@pytest.mark.parametrize("module,flavor", FAMILIES)
def test_family_on_kernels_matches_cpu_reference(module, flavor):
    try:
        spec = get_model_spec(module, flavor)
    except ValueError:
        pytest.skip(f"{module} has no flavor {flavor}")
    torch.manual_seed(0)
    ref = spec.model.build()
    ref.init_states(seed=11)
    ref = ref.float()
    with torch.no_grad():                      # parameters that start at zero (offset gains, gated outputs) get a signal
        for p in ref.parameters():
            if float(p.abs().max()) == 0.0:
                p.normal_(std=0.05)
    T = 160
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, spec.model.vocab_size, (T + 1,), generator=g)
    tok, lab = ids[:-1], ids[1:]
    pos = torch.arange(T)
    pos[96:] -= 96                                 # two documents: 96 + 64 tokens
    logits_ref = ref(tok, pos)
    loss_ref = torch.nn.functional.cross_entropy(logits_ref.float(), lab, reduction="sum") / T
    loss_ref.backward()

    dev = torch.device("cuda")
    model = copy.deepcopy(ref)
    model.zero_grad(set_to_none=True)
    model.to(dev)
    for p in model.parameters():
        p.data = p.data.to(torch.bfloat16)
    before = OF.settings.library_fallbacks
    logits = model(tok.to(dev), pos.to(dev))
    loss = torch.nn.functional.cross_entropy(logits.float(), lab.to(dev), reduction="sum") / T
    loss.backward()
    torch.cuda.synchronize()
    assert torch.isfinite(logits).all()
    scale = float(logits_ref.detach().abs().max())
    err = float((logits.detach().float().cpu() - logits_ref.detach()).abs().max())
    assert err <= 0.06 * scale + 0.06, (err, scale, OF.settings.library_fallbacks - before)
    assert abs(float(loss) - float(loss_ref)) <= 0.03 * abs(float(loss_ref)) + 0.03, (float(loss), float(loss_ref))
    ge, gr = model.tok_embeddings.weight.grad.float().cpu(), ref.tok_embeddings.weight.grad
    assert torch.isfinite(ge).all()
    cos = float((ge * gr).sum() / (ge.norm() * gr.norm() + 1e-12))
    # muse_glimmer multiplies unit-norm queries by 5.5: attention scores reach +-40 and bf16 rounding of q / k alone moves
    # the gradient this far (the CPU reference run in bf16 against itself in fp32 gives the same 0.76)
    assert cos > (0.6 if module == "muse_glimmer" else 0.98), cos
