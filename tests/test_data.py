"""Data pipeline: batch contract, packing modes, resume exactness, dp sharding, SFT masking, tokenizer."""

import os

import pytest
import torch

from torchtitan_b200.components.data import BaseDataLoader, SyntheticDataLoader
from torchtitan_b200.components.data.text import TextDataLoader
from torchtitan_b200.components.tokenizer import ByteTokenizer, HuggingFaceTokenizer

ASSETS = os.path.join(os.path.dirname(__file__), "assets")


@pytest.fixture(scope="module")
def tok():
    return HuggingFaceTokenizer(tokenizer_path=os.path.join(ASSETS, "tokenizer"))


def _loader(tok, dataset="c4_test", T=256, ctx=128, rank=0, world=1, **kw):
    cfg = BaseDataLoader.Config(dataset=dataset, pin_memory=False, **kw)
    return cfg.build(dp_world_size=world, dp_rank=rank, num_tokens_per_batch=T, max_context_length=ctx, tokenizer=tok)


def test_tokenizer_bos_eos(tok):
    ids = tok.encode("The river crosses the quiet valley.")
    assert ids[0] == tok.bos_id and ids[-1] == tok.eos_id
    plain = tok.encode("The river crosses the quiet valley.", add_bos=False, add_eos=False)
    assert plain == ids[1:-1]
    assert tok.decode(plain) == "The river crosses the quiet valley."
    assert tok.get_vocab_size() > 256


def test_build_dispatches_on_dataset_name(tok):
    assert isinstance(_loader(tok), TextDataLoader)
    syn = BaseDataLoader.Config(dataset="synthetic", pin_memory=False).build(num_tokens_per_batch=64, vocab_size=100)
    assert isinstance(syn, SyntheticDataLoader)
    (inp, lab) = next(iter(syn))
    assert inp["input"].shape == (64,) and lab.shape == (64,) and int(inp["input"].max()) < 100
    assert torch.equal(inp["input"][1:], lab[:-1])


def test_concat_packing_contract(tok):
    it = iter(_loader(tok))
    for _ in range(5):
        inp, lab = next(it)
        assert inp["input"].shape == (256,) and inp["positions"].shape == (256,) and lab.shape == (256,)
        pos = inp["positions"]
        assert pos[0] == 0 and int(pos.max()) < 128
        # positions increase by one inside a piece and restart at zero
        d = pos[1:] - pos[:-1]
        assert ((d == 1) | (pos[1:] == 0)).all()
        # labels are next tokens inside a piece
        same_piece = d == 1
        assert torch.equal(inp["input"][1:][same_piece], lab[:-1][same_piece])


def test_first_fit_never_splits_and_pads(tok):
    it = iter(_loader(tok, packing="first_fit", num_packing_bins=4, T=300))
    saw_pad = False
    for _ in range(6):
        inp, lab = next(it)
        pos = inp["positions"]
        assert pos[0] == 0
        pad = lab == -100
        n = int((~pad).sum())
        if n < 300:
            saw_pad = True
            assert (inp["input"][n:] == 0).all() and pos[n] == 0
    assert saw_pad


def test_resume_reproduces_stream(tok):
    a = _loader(tok)
    it = iter(a)
    for _ in range(3):
        next(it)
    state = a.state_dict()
    expect = [next(it) for _ in range(4)]
    b = _loader(tok)
    b.load_state_dict(state)
    it2 = iter(b)
    for e in expect:
        g = next(it2)
        assert torch.equal(e[0]["input"], g[0]["input"]) and torch.equal(e[1], g[1])
    with pytest.raises(ValueError):
        _loader(tok, world=2).load_state_dict(state)


def test_dp_ranks_read_disjoint_samples(tok):
    a, b = _loader(tok, rank=0, world=2), _loader(tok, rank=1, world=2)
    assert not set(a._epoch_indices()) & set(b._epoch_indices())


def test_finite_loader_stops(tok):
    n = sum(1 for _ in _loader(tok, repeat=False, shuffle=False, T=4096, ctx=512))
    assert 2 < n < 100


def test_sft_masks_prompt(tok):
    inp, lab = next(iter(_loader(tok, dataset="sft_test", T=128, ctx=128)))
    assert (lab == -100).any() and (lab != -100).any()
    first_doc_end = (inp["positions"][1:] == 0).nonzero().flatten()[0].item() + 1
    seg = lab[:first_doc_end]
    k = (seg != -100).nonzero().flatten()[0].item()
    assert (seg[:k] == -100).all() and (seg[k:] != -100).all()


def test_byte_tokenizer_round_trip():
    t = ByteTokenizer()
    ids = t.encode("héllo")
    assert t.decode(ids) == "héllo" and ids[0] == t.bos_id


def test_concat_and_mix_datasets(tok):
    from torchtitan_b200.components.data.text import DATASETS, ConcatSource, MixSource, parse_composite

    assert parse_composite("mix:c4_test=0.75,sft_test=0.25") == ("mix", ["c4_test", "sft_test"], [0.75, 0.25])
    a, b = DATASETS["c4_test"].make_source(None), DATASETS["sft_test"].make_source(None)
    cat = ConcatSource([a, b])
    assert len(cat) == len(a) + len(b) and cat[0]["__dataset__"] == 0 and cat[len(a)]["__dataset__"] == 1
    assert "text" in cat[0] and "question" in cat[len(a)]
    mix = MixSource([a, b], [0.75, 0.25], seed=3)
    picks = [mix[i]["__dataset__"] for i in range(len(mix))]
    assert 0 < sum(picks) < len(picks)                     # both datasets appear
    assert picks == [MixSource([a, b], [0.75, 0.25], seed=3)[i]["__dataset__"] for i in range(len(mix))]
    # through the loader: SFT samples carry masked prompts, plain text does not
    for name in ("concat:c4_test,sft_test", "mix:c4_test=0.5,sft_test=0.5"):
        it = iter(_loader(tok, dataset=name, shuffle=True))
        seen_masked = False
        for _ in range(12):
            inp, lab = next(it)
            assert inp["input"].shape == (256,)
            seen_masked |= bool(((lab == -100) & (inp["positions"] > 0)).any())
        assert seen_masked
    with pytest.raises(ValueError):
        _loader(tok, dataset="mix:c4_test=1,nope=1")
