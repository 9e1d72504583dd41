"""Vision tower, placeholder scattering, three-axis rotary positions and the multimodal collator."""

import pytest
import torch

from torchtitan_b200.components.data.multimodal import MultimodalCollator, patchify
from torchtitan_b200.models.common.layers import RoPE
from torchtitan_b200.models.common.multimodal import get_vision_positions, mrope_position_ids, scatter_vision_embeds
from torchtitan_b200.models.common.vision_encoder import VisionEncoder, rope_2d
from torchtitan_b200.ops.reference import IGNORE_INDEX


def test_patchify_and_collator():
    img = torch.arange(3 * 8 * 12, dtype=torch.float32).reshape(3, 8, 12)
    p, (gh, gw) = patchify(img, patch=2, merge=2)
    assert (gh, gw) == (4, 6) and p.shape == (24, 12)
    assert torch.equal(p[7].reshape(3, 2, 2), img[:, 2:4, 2:4])          # patch (row 1, col 1)
    col = MultimodalCollator(32, patch=2, merge=2, image_token_id=99, max_context_length=32)
    a, b, patches, grids = col.encode([[1, 2, 3], img, [4, 5]])
    assert a == [1, 2, 3] + [99] * 6 + [4] and grids == [(4, 6)]
    assert b == [2, 3] + [IGNORE_INDEX] * 6 + [4, 5]                      # image slots are never targets
    batch, labels = col.collate([(a, b, patches, grids)])
    assert batch["input"].shape == (32,) and batch["pixel_patches"].shape == (24, 12)
    assert batch["grid_hw"].tolist() == [[4, 6]] and batch["positions"][:12].tolist() == list(range(10)) + [0, 1]
    assert (labels[10:] == IGNORE_INDEX).all()


def test_scatter_and_alignment_errors():
    tok = torch.tensor([5, 9, 9, 6, 9, 7])
    pos = get_vision_positions(tok, torch.tensor([2, 1]), 9)
    assert pos == [(0, 1, 2), (1, 4, 1)]
    emb = torch.zeros(6, 4, requires_grad=True)
    vis = torch.ones(3, 4, requires_grad=True)
    out = scatter_vision_embeds(emb, vis, pos)
    assert out[:, 0].tolist() == [0, 1, 1, 0, 1, 0]
    out.sum().backward()
    assert vis.grad.sum() == 12 and emb.grad[1].sum() == 0 and emb.grad[0].sum() == 4
    with pytest.raises(ValueError):
        get_vision_positions(tok, torch.tensor([2]), 9)
    with pytest.raises(ValueError):
        get_vision_positions(tok, torch.tensor([1, 1]), 9)


def test_mrope_positions_and_table():
    tok = torch.tensor([1, 2, 9, 9, 9, 9, 3, 4, 1, 2])
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 0, 1])
    ids = mrope_position_ids(tok, pos, torch.tensor([[4, 4]]), 2, 9)
    assert ids[0].tolist() == [0, 1, 2, 2, 2, 2, 4, 5, 0, 1]
    assert ids[1].tolist() == [0, 1, 2, 2, 3, 3, 4, 5, 0, 1]
    assert ids[2].tolist() == [0, 1, 2, 3, 2, 3, 4, 5, 0, 1]
    rope = RoPE.Config(dim=16, max_context_length=64, style="cos_sin", mrope_sections=(4, 2, 2)).build()
    rope.init_buffers(torch.device("cpu"))
    x = torch.randn(10, 2, 16)
    # identical axes reproduce ordinary RoPE
    same = pos.unsqueeze(0).expand(3, -1)
    assert torch.allclose(rope(x, same), rope(x, pos), atol=1e-6)
    # frequency f follows its section's axis
    table, _ = rope._table_for(ids)
    assert torch.equal(table[3, 0:4], rope.cache[2, 0:4]) and torch.equal(table[4, 4:6], rope.cache[3, 4:6])
    assert torch.equal(table[3, 6:8], rope.cache[3, 6:8]) and torch.equal(table[3, 8 + 6:8 + 8], rope.cache[3, 8 + 6:8 + 8])


def test_vision_encoder_is_block_diagonal_and_position_aware():
    torch.manual_seed(0)
    enc = VisionEncoder.Config(patch_size=2, dim=32, num_heads=2, mlp_dim=64, n_layers=2, spatial_merge=2, out_dim=48).build()
    enc.init_states(seed=1)
    a, b = torch.randn(16, 12), torch.randn(8, 12)
    both, n = enc(torch.cat([a, b]), torch.tensor([[4, 4], [2, 4]]))
    assert both.shape == (4 + 2, 48) and n.tolist() == [4, 2]
    only_a, _ = enc(a, torch.tensor([[4, 4]]))
    assert torch.allclose(both[:4], only_a, atol=1e-5)        # the second image does not leak into the first
    x = torch.randn(4, 2, 16)
    r = rope_2d(x, torch.tensor([0, 0, 1, 1]), torch.tensor([0, 1, 0, 1]))
    assert torch.allclose(r[0], x[0]) and not torch.allclose(r[3], x[3])
    assert torch.allclose(r.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_qwen3_5_vision_language_matches_transformers():
    """The vision-language flavor on weights taken from a freshly initialised ``Qwen3_5ForConditionalGeneration``: the
    ViT tower (two-frame patch embedding, interpolated position table, 2-D rotary attention, 2 x 2 merger), the
    placeholder scatter, the three-axis position rule and the interleaved multimodal RoPE give transformers' logits
    on text interleaved with two images; the adapter's visual names round-trip."""
    import pytest

    pytest.importorskip("transformers")
    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.scripts.numerical_tests import main

    res = main(["--module", "qwen3_5", "--flavor", "debugmodel_vl", "--random", "--perturb", "0.1"])
    assert abs(res["kl_mean"]) < 1e-6 and res["max_abs_logit_diff"] < 1e-4, res

    spec = get_model_spec("qwen3_5", "debugmodel_vl")
    model = spec.model.build()
    model.init_states(seed=2)
    ad = spec.state_dict_adapter(spec.model, None)
    vis = {k: p.detach() for k, p in model.named_parameters() if k.startswith("vision_encoder.")}
    hf = ad.to_hf(dict(vis))
    assert hf["model.visual.patch_embed.proj.weight"].dim() == 5 and "model.visual.blocks.0.attn.qkv.weight" in hf
    back = ad.from_hf(hf)
    assert set(back) == set(vis) and all(torch.equal(back[k], vis[k]) for k in vis)
