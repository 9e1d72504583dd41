"""Text datasets: sources -> sample processors -> packing -> fixed-size token batches.

Pipeline (parity: torchtitan/components/data/{sources,dataset,packing,collators,loader}.py and
hf_datasets/text_datasets.py):

* **source**: random-access JSONL files (byte-offset index built once) or a Hugging Face dataset
  (map-style or streaming).  Each dp rank reads a disjoint contiguous slice of the (per-epoch
  shuffled) index space; streaming sources are read round-robin with a window shuffle.
* **processor**: ``TextProcessor`` encodes ``text`` with BOS/EOS; ``ChatProcessor`` renders one
  prompt/response turn with the tokenizer's chat template and masks the prompt labels.
  A sample is ``ids[:-1]`` (inputs) and ``ids[1:]`` (labels).
* **packing**: ``concat`` streams document pieces (at most ``max_context_length`` tokens each)
  back to back into batches of exactly ``T`` tokens; ``first_fit`` keeps ``num_packing_bins`` open
  bins, never splits a piece and pads the emitted bin (token 0, label -100, fresh positions).
  ``positions`` restart at 0 at every piece, which is what the attention mask keys on.
* **state**: epoch, cursor inside the epoch's permutation, and the packer's carry-over; restoring
  it reproduces the token stream exactly.  A state saved with another dp degree is refused.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Iterator

import torch

from torchtitan_b200.components.loss import IGNORE_INDEX
from torchtitan_b200.utils.logging import logger

from .loader import BaseDataLoader

__all__ = ["TextDataLoader", "DATASETS", "DatasetSpec", "JsonlSource", "HuggingFaceSource", "TextProcessor",
           "ChatProcessor", "register_dataset", "ConcatSource", "MixSource"]

_ASSETS = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))),
                       "tests", "assets")


# ----------------------------------------------------------------------------
# sources
# ----------------------------------------------------------------------------
class JsonlSource:
    """Random access over the lines of one or more ``.jsonl`` / ``.json`` (one object per line) files."""

    random_access = True

    def __init__(self, patterns: tuple[str, ...] | list[str]):
        import glob

        self.files = sorted(f for p in patterns for f in glob.glob(p))
        if not self.files:
            raise FileNotFoundError(f"no files match {patterns}")
        self.index: list[tuple[int, int]] = []
        for fi, path in enumerate(self.files):
            off = 0
            with open(path, "rb") as f:
                for line in f:
                    if line.strip():
                        self.index.append((fi, off))
                    off += len(line)
        self._handles: dict[int, Any] = {}

    def __len__(self) -> int:
        return len(self.index)

    def __getitem__(self, i: int) -> dict:
        fi, off = self.index[i]
        h = self._handles.get(fi)
        if h is None:
            h = self._handles[fi] = open(self.files[fi], "rb")
        h.seek(off)
        return json.loads(h.readline())


class HuggingFaceSource:
    """A Hugging Face dataset: map-style (random access) or streaming."""

    def __init__(self, path: str, split: str, name: str | None = None, streaming: bool = False,
                 revision: str | None = None, **load_kwargs):
        from datasets import load_dataset

        self.random_access = not streaming
        self.ds = load_dataset(path, name=name, split=split, streaming=streaming, revision=revision, **load_kwargs)

    def __len__(self) -> int:
        return len(self.ds)

    def __getitem__(self, i: int) -> dict:
        return self.ds[int(i)]

    def iter_from(self, skip: int, shard_rank: int, shard_world: int) -> Iterator[dict]:
        ds = self.ds
        if hasattr(ds, "shard") and shard_world > 1:
            try:
                ds = ds.shard(num_shards=shard_world, index=shard_rank)
                shard_world = 1
            except Exception:
                pass
        for i, sample in enumerate(ds):
            if shard_world > 1 and i % shard_world != shard_rank:
                continue
            if skip > 0:
                skip -= 1
                continue
            yield sample


# ----------------------------------------------------------------------------
# processors
# ----------------------------------------------------------------------------
class TextProcessor:
    def __init__(self, tokenizer, text_key: str = "text", add_bos: bool = True, add_eos: bool = True):
        self.tok, self.key, self.add_bos, self.add_eos = tokenizer, text_key, add_bos, add_eos

    def __call__(self, sample: dict):
        ids = self.tok.encode(sample[self.key], add_bos=self.add_bos, add_eos=self.add_eos)
        if len(ids) < 2:
            return None
        return ids[:-1], ids[1:]


class ChatProcessor:
    """Single-turn SFT: the prompt part of the rendered conversation gets label -100."""

    def __init__(self, tokenizer, prompt_key: str = "question", response_key: str = "answer"):
        self.tok, self.pk, self.rk = tokenizer, prompt_key, response_key

    def _render(self, messages, add_generation_prompt):
        if getattr(self.tok, "chat_template", None):
            return self.tok.apply_chat_template(messages, add_generation_prompt=add_generation_prompt)
        text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages)
        return text + ("<|assistant|>\n" if add_generation_prompt else "")

    def __call__(self, sample: dict):
        prompt = [{"role": "user", "content": sample[self.pk]}]
        full = prompt + [{"role": "assistant", "content": sample[self.rk]}]
        p_ids = self.tok.encode(self._render(prompt, True), add_bos=True, add_eos=False)
        f_ids = self.tok.encode(self._render(full, False), add_bos=True, add_eos=True)
        if len(f_ids) < 2:
            return None
        n_prompt = min(len(p_ids), len(f_ids) - 1)
        labels = list(f_ids[1:])
        for i in range(max(0, n_prompt - 1)):
            labels[i] = IGNORE_INDEX
        return f_ids[:-1], labels


# ----------------------------------------------------------------------------
# registry
# ----------------------------------------------------------------------------
@dataclass
class DatasetSpec:
    make_source: Callable[[str | None], Any]
    make_processor: Callable[[Any], Callable[[dict], Any]]


def _c4(split: str, streaming: bool = True):
    return lambda path: HuggingFaceSource(path or "allenai/c4", split=split, name="en", streaming=streaming)


DATASETS: dict[str, DatasetSpec] = {
    "c4": DatasetSpec(_c4("train"), lambda tok: TextProcessor(tok)),
    "c4_validation": DatasetSpec(_c4("validation"), lambda tok: TextProcessor(tok)),
    "c4_test": DatasetSpec(lambda path: JsonlSource([os.path.join(path or os.path.join(_ASSETS, "c4_test"), "*.json*")]),
                           lambda tok: TextProcessor(tok)),
    "sft_test": DatasetSpec(lambda path: JsonlSource([os.path.join(path or os.path.join(_ASSETS, "sft_test"), "*.json*")]),
                            lambda tok: ChatProcessor(tok)),
}


def register_dataset(name: str, spec: DatasetSpec) -> None:
    DATASETS[name] = spec


# ----------------------------------------------------------------------------
# composite datasets
# ----------------------------------------------------------------------------
class ConcatSource:
    """Several random-access sources end to end; samples carry the index of their dataset so
    that each goes through its own processor."""

    random_access = True

    def __init__(self, sources: list):
        if not all(getattr(s, "random_access", True) for s in sources):
            raise ValueError("composite datasets need random-access (non-streaming) sources")
        self.sources = sources
        self.starts = [0]
        for src in sources:
            self.starts.append(self.starts[-1] + len(src))

    def __len__(self) -> int:
        return self.starts[-1]

    def __getitem__(self, i: int) -> dict:
        import bisect

        k = bisect.bisect_right(self.starts, i) - 1
        return {"__dataset__": k, **self.sources[k][i - self.starts[k]]}


class MixSource(ConcatSource):
    """Weighted interleave: position i of the (virtual) epoch draws its dataset from the
    normalised weights with a fixed seed and takes that dataset's next sample, wrapping around a
    dataset that is exhausted (small datasets repeat, large ones are subsampled).  The epoch has
    as many positions as all datasets together."""

    def __init__(self, sources: list, weights: list[float], seed: int = 0):
        super().__init__(sources)
        if len(weights) != len(sources) or min(weights) <= 0:
            raise ValueError("a dataset mix needs one positive weight per dataset")
        n = self.starts[-1]
        g = torch.Generator().manual_seed(seed)
        pick = torch.multinomial(torch.tensor(weights, dtype=torch.float64), n, replacement=True, generator=g)
        self.pick = pick.tolist()
        counts = [0] * len(sources)
        self.local = []
        for k in self.pick:
            self.local.append(counts[k] % len(sources[k]))
            counts[k] += 1

    def __getitem__(self, i: int) -> dict:
        k = self.pick[i]
        return {"__dataset__": k, **self.sources[k][self.local[i]]}


def parse_composite(name: str):
    """``concat:a,b`` -> ("concat", [a, b], None);  ``mix:a=0.7,b=0.3`` -> ("mix", [a, b], [0.7, 0.3])."""
    kind, _, rest = name.partition(":")
    parts = [x for x in rest.split(",") if x]
    if kind == "concat":
        return kind, parts, None
    names, weights = [], []
    for part in parts:
        n, _, w = part.partition("=")
        names.append(n)
        weights.append(float(w) if w else 1.0)
    return kind, names, weights


# ----------------------------------------------------------------------------
# loader
# ----------------------------------------------------------------------------
class TextDataLoader(BaseDataLoader):
    def __init__(self, config: BaseDataLoader.Config, *, dp_world_size: int = 1, dp_rank: int = 0,
                 num_tokens_per_batch: int = 2048, max_context_length: int = 2048, vocab_size: int = 0,
                 tokenizer=None, **_):
        self.config = config
        if tokenizer is None:
            raise ValueError("a tokenizer is required for text datasets")
        if config.dataset.startswith(("mix:", "concat:")):
            # composite: ``concat:a,b`` or ``mix:a=0.7,b=0.3`` over registered datasets
            # (parity: DatasetConcatConfig / DatasetMixConfig of torchtitan/components/data/dataset.py:197-309)
            kind, names, weights = parse_composite(config.dataset)
            unknown = [n for n in names if n not in DATASETS]
            if unknown or not names:
                raise ValueError(f"unknown dataset(s) {unknown} in '{config.dataset}' (registered: {sorted(DATASETS)})")
            sources = [DATASETS[n].make_source(None) for n in names]
            procs = [DATASETS[n].make_processor(tokenizer) for n in names]
            self.source = ConcatSource(sources) if kind == "concat" else MixSource(sources, weights, seed=config.seed)
            self.process = lambda sample: procs[sample["__dataset__"]](sample)
        else:
            if config.dataset not in DATASETS:
                raise ValueError(f"unknown dataset '{config.dataset}' (registered: {sorted(DATASETS)})")
            spec = DATASETS[config.dataset]
            self.source = spec.make_source(config.dataset_path)
            self.process = spec.make_processor(tokenizer)
        self.dp_world_size, self.dp_rank = dp_world_size, dp_rank
        self.T, self.ctx = num_tokens_per_batch, min(max_context_length, num_tokens_per_batch)
        self.epoch = 0
        self.cursor = 0  # samples consumed in this epoch by this rank
        self.carry: list[tuple[list[int], list[int]]] = []  # packer leftovers (inputs, labels) pieces
        self.bins: list[list[tuple[list[int], list[int]]]] = []
        self.pin = config.pin_memory and torch.cuda.is_available()
        logger.info(f"Preparing dataset {config.dataset} for dp rank {dp_rank}/{dp_world_size}")

    # -- sample stream -----------------------------------------------------------
    def _epoch_indices(self) -> list[int]:
        n = len(self.source)
        if self.config.shuffle:
            g = torch.Generator().manual_seed(self.config.seed + self.epoch)
            perm = torch.randperm(n, generator=g).tolist()
        else:
            perm = list(range(n))
        per = n // self.dp_world_size
        if per == 0:
            raise ValueError(f"dataset has {n} samples, fewer than the dp degree {self.dp_world_size}")
        return perm[self.dp_rank * per:(self.dp_rank + 1) * per]

    def _samples(self) -> Iterator[dict]:
        while True:
            if getattr(self.source, "random_access", True):
                idx = self._epoch_indices()
                while self.cursor < len(idx):
                    i = idx[self.cursor]
                    self.cursor += 1
                    yield self.source[i]
            else:
                buf: list[dict] = []
                g = torch.Generator().manual_seed(self.config.seed + self.epoch * 7919 + self.dp_rank)
                window = 1000 if self.config.shuffle else 1
                for s in self.source.iter_from(self.cursor, self.dp_rank, self.dp_world_size):
                    self.cursor += 1
                    buf.append(s)
                    if len(buf) >= window:
                        yield buf.pop(int(torch.randint(len(buf), (1,), generator=g)))
                while buf:
                    yield buf.pop(int(torch.randint(len(buf), (1,), generator=g)))
            if not self.config.repeat:
                return
            self.epoch += 1
            self.cursor = 0
            logger.warning(f"Dataset {self.config.dataset} is being re-looped (epoch {self.epoch})")

    def _docs(self) -> Iterator[tuple[list[int], list[int]]]:
        for sample in self._samples():
            out = self.process(sample)
            if out is not None:
                yield list(out[0]), list(out[1])

    # -- batch assembly ------------------------------------------------------------
    def _emit(self, pieces: list[tuple[list[int], list[int]]]):
        T = self.T
        inp = torch.zeros(T, dtype=torch.int64)
        lab = torch.full((T,), IGNORE_INDEX, dtype=torch.int64)
        pos = torch.zeros(T, dtype=torch.int64)
        o = 0
        for a, b in pieces:
            n = len(a)
            inp[o:o + n] = torch.tensor(a, dtype=torch.int64)
            lab[o:o + n] = torch.tensor(b, dtype=torch.int64)
            pos[o:o + n] = torch.arange(n)
            o += n
        if o < T:
            pos[o:] = torch.arange(T - o)  # padding behaves like one more (ignored) document
        if self.pin:
            inp, lab, pos = inp.pin_memory(), lab.pin_memory(), pos.pin_memory()
        return {"input": inp, "positions": pos}, lab

    def _with_carry(self) -> Iterator[tuple[list[int], list[int]]]:
        """Unfinished work restored from a checkpoint comes first, then fresh documents."""
        pending, self.carry = self.carry, []
        yield from pending
        yield from self._docs()

    def _concat_batches(self):
        # ``carry`` = the not yet consumed tail of the current document.  When a batch fills in
        # the middle of a document the tail is treated as a new document (positions restart),
        # both in an uninterrupted run and after a restore, so the two produce the same stream.
        cur: list[tuple[list[int], list[int]]] = []
        fill = 0
        for a, b in self._with_carry():
            while a:
                take = min(self.T - fill, self.ctx, len(a))
                cur.append((a[:take], b[:take]))
                fill += take
                a, b = a[take:], b[take:]
                if fill == self.T:
                    self.carry = [(a, b)] if a else []
                    yield self._emit(cur)
                    self.carry = []
                    cur, fill = [], 0
        if cur:
            yield self._emit(cur)

    def _first_fit_batches(self):
        nb = max(1, self.config.num_packing_bins)
        for a, b in self._with_carry():
            pieces = [(a[s:s + self.ctx], b[s:s + self.ctx]) for s in range(0, len(a), self.ctx)]
            for i, (pa, pb) in enumerate(pieces):
                placed = False
                for bin_ in self.bins:
                    if sum(len(x) for x, _ in bin_) + len(pa) <= self.T:
                        bin_.append((pa, pb))
                        placed = True
                        break
                if placed:
                    continue
                if len(self.bins) >= nb:
                    fullest = max(range(len(self.bins)), key=lambda j: sum(len(x) for x, _ in self.bins[j]))
                    out = self.bins.pop(fullest)
                    self.carry = [(sum((p[0] for p in pieces[i:]), []), sum((p[1] for p in pieces[i:]), []))]
                    yield self._emit(out)
                    self.carry = []
                self.bins.append([(pa, pb)])
        while self.bins:
            yield self._emit(self.bins.pop(0))

    def __iter__(self):
        if self.config.packing == "first_fit":
            return self._first_fit_batches()
        return self._concat_batches()

    # -- state -----------------------------------------------------------------------
    def state_dict(self):
        return {"version": 1, "dp_world_size": self.dp_world_size,
                f"dp_rank_{self.dp_rank}": {"epoch": self.epoch, "cursor": self.cursor,
                                            "carry": json.dumps(self.carry), "bins": json.dumps(self.bins)}}

    def load_state_dict(self, sd):
        if not sd:
            return
        if sd.get("dp_world_size", self.dp_world_size) != self.dp_world_size:
            raise ValueError(f"dataloader state was saved with dp degree {sd.get('dp_world_size')}, cannot resume "
                             f"with {self.dp_world_size}")
        st = sd.get(f"dp_rank_{self.dp_rank}")
        if st is None:
            return
        self.epoch, self.cursor = int(st["epoch"]), int(st["cursor"])
        self.carry = [(list(a), list(b)) for a, b in json.loads(st["carry"])]
        self.bins = [[(list(a), list(b)) for a, b in bin_] for bin_ in json.loads(st["bins"])]
