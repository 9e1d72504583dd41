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


def test_media_fit_to_grid_image_and_video(tmp_path):
    """Sizes land on the patch grid inside the pixel budget; an image file and a video file written here decode, and a
    JSONL sample with text, an image and a video becomes placeholder runs of the right lengths."""
    import json

    import numpy as np

    from torchtitan_b200.components.data import media

    for (h, w) in [(480, 640), (33, 1000), (2000, 3000), (20, 20)]:
        H, W = media.fit_to_grid(h, w, factor=28, min_pixels=56 * 56, max_pixels=512 * 512)
        assert H % 28 == 0 and W % 28 == 0 and 56 * 56 <= H * W <= 512 * 512 + 28 * 28 * 4
    assert media.fit_to_grid(448, 448, factor=28, min_pixels=1, max_pixels=10 ** 9) == (448, 448)
    with pytest.raises(ValueError):
        media.fit_to_grid(1, 1000, factor=28, min_pixels=1, max_pixels=10 ** 6)
    assert media.sample_frame_indices(100, 25.0, fps=2.0, min_frames=4, max_frames=768) == [0, 14, 28, 42, 57, 71, 85, 99]
    assert media.sample_frame_indices(3, 30.0, min_frames=4) == [0, 1, 2]
    assert len(media.sample_frame_indices(10000, 25.0, fps=2.0, max_frames=16)) == 16

    from PIL import Image

    rng = np.random.default_rng(0)
    img_path = str(tmp_path / "a.png")
    Image.fromarray(rng.integers(0, 255, (70, 90, 3), dtype=np.uint8)).save(img_path)
    img = media.load_image(img_path)
    assert img.shape == (3, 70, 90) and img.dtype == torch.uint8
    out = media.process_image(img, patch_size=4, merge_size=2, min_pixels=64, max_pixels=48 * 48)
    assert out.dtype == torch.float32 and out.shape[1] % 8 == 0 and out.shape[2] % 8 == 0 and out.abs().max() <= 1.0 + 1e-5

    cv2 = pytest.importorskip("cv2")
    vid_path = str(tmp_path / "v.avi")
    wr = cv2.VideoWriter(vid_path, cv2.VideoWriter_fourcc(*"MJPG"), 10.0, (64, 48))
    if not wr.isOpened():
        pytest.skip("no MJPG encoder in this OpenCV build")
    for i in range(20):
        wr.write(np.full((48, 64, 3), i * 10, dtype=np.uint8))
    wr.release()
    clip = media.load_video(vid_path, fps=2.0, min_frames=4, max_frames=8)
    assert clip is not None and clip.shape == (4, 48, 64, 3)          # 2 s at 2 fps, raised to the minimum of 4 frames
    assert clip[0].float().mean() < clip[-1].float().mean()            # frames come in order
    frames = media.process_video(clip, patch_size=4, merge_size=2, min_pixels=64, max_pixels=32 * 32)
    assert frames.shape[0] == 4 and frames.shape[1] == 3 and frames.shape[2] % 8 == 0 and frames.shape[3] % 8 == 0
    assert media.load_video(str(tmp_path / "missing.mp4")) is None

    from torchtitan_b200.components.data import BaseDataLoader
    from torchtitan_b200.components.data.multimodal import MultimodalDataLoader
    from torchtitan_b200.components.tokenizer import ByteTokenizer

    jl = tmp_path / "mm.jsonl"
    jl.write_text(json.dumps({"segments": [{"text": "look:"}, {"image": img_path}, {"text": "then"},
                                           {"video": vid_path, "max_frames": 4, "max_pixels": 32 * 32}]}) + "\n")
    dl = MultimodalDataLoader(BaseDataLoader.Config(dataset="mm_jsonl", dataset_path=str(jl)), num_tokens_per_batch=4096,
                              max_context_length=4096, tokenizer=ByteTokenizer(), patch_size=4, spatial_merge=2,
                              image_token_id=300)
    batch, labels = next(iter(dl))
    grids = batch["grid_hw"]
    assert grids.shape[0] >= 5                                          # one image and four frames (per packed sample)
    n_slots = int((batch["input"] == 300).sum()) + int(batch["input"][0] == 300)
    assert n_slots >= int((grids[:5, 0] * grids[:5, 1] // 4).sum()) - 1
    assert batch["pixel_patches"].shape[1] == 3 * 4 * 4
