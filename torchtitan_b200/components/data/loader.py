"""Data loaders.

Batch contract (parity: torchtitan/components/data/collators.py:52-79): every
iteration yields ``({"input": int64[T], "positions": int64[T]}, labels int64[T])`` on
the CPU, with ``T = training.num_tokens_per_microbatch_per_dp_rank``.  Documents are
packed; ``positions`` restart at 0 at each document start; padding uses token 0,
label ``-100`` and fresh positions.

Loaders are stateful (``state_dict`` / ``load_state_dict``) and keyed by dp rank; a
checkpoint taken with another dp degree is refused (parity: data/loader.py:161-164).
"""

from __future__ import annotations

import queue
import threading
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch

from torchtitan_b200.config import Configurable

__all__ = ["BaseDataLoader", "SyntheticDataLoader", "DataloaderExhaustedError", "PrefetchIterator"]


class DataloaderExhaustedError(Exception):
    """Raised when a finite dataloader has no more batches; the trainer ends the run cleanly."""


class BaseDataLoader(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        dataset: str = "synthetic"
        """``synthetic``, ``synthetic_mm`` / ``mm_jsonl`` (interleaved text and images) or the name of
        a registered text dataset (``c4``, ``c4_test`` ...)."""
        dataset_path: str | None = None
        seed: int = 42
        shuffle: bool = True
        repeat: bool = True
        num_prefetch_batches: int = 2
        packing: str = "concat"  # concat | first_fit
        num_packing_bins: int = 8
        synthetic_vocab_size: int | None = None
        synthetic_doc_len: int | None = None
        """Document length of synthetic data (``None`` = ``max_context_length``)."""
        pin_memory: bool = True

    def __new__(cls, config=None, **kw):
        if cls is BaseDataLoader and config is not None:
            if config.dataset == "synthetic":
                return object.__new__(SyntheticDataLoader)
            if config.dataset in ("synthetic_mm", "mm_jsonl"):
                from .multimodal import MultimodalDataLoader

                return object.__new__(MultimodalDataLoader)
            from .text import TextDataLoader

            return object.__new__(TextDataLoader)
        return object.__new__(cls)

    def __iter__(self) -> Iterator:
        raise NotImplementedError

    def state_dict(self) -> dict[str, Any]:
        return {}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        pass


class SyntheticDataLoader(BaseDataLoader):
    """Uniform-random token ids; labels are the tokens shifted by one.

    The stream of dp rank ``r`` at batch ``i`` is a pure function of
    ``(seed, r, i)``: resuming only needs the batch counter.
    """

    def __init__(self, config: BaseDataLoader.Config, *, dp_world_size: int = 1, dp_rank: int = 0,
                 num_tokens_per_batch: int = 2048, max_context_length: int = 2048, vocab_size: int = 2048,
                 tokenizer=None, **_):
        self.config = config
        self.dp_world_size, self.dp_rank = dp_world_size, dp_rank
        self.T = num_tokens_per_batch
        self.doc_len = min(config.synthetic_doc_len or max_context_length, max_context_length)
        self.vocab = config.synthetic_vocab_size or vocab_size
        self.batch_idx = 0
        self.pin = config.pin_memory and torch.cuda.is_available()

    def _make(self, idx: int):
        g = torch.Generator()
        g.manual_seed((self.config.seed * 1_000_003 + self.dp_rank) * 1_000_003 + idx)
        T = self.T
        n_docs = -(-T // self.doc_len)
        ids = torch.randint(0, self.vocab, (T + n_docs,), generator=g, dtype=torch.int64)
        inp = torch.empty(T, dtype=torch.int64)
        lab = torch.empty(T, dtype=torch.int64)
        pos = torch.empty(T, dtype=torch.int64)
        o = 0
        for d in range(n_docs):
            n = min(self.doc_len, T - o)
            doc = ids[d * (self.doc_len + 1): d * (self.doc_len + 1) + n + 1]
            inp[o:o + n] = doc[:-1]
            lab[o:o + n] = doc[1:]
            pos[o:o + n] = torch.arange(n)
            o += n
        if self.pin:
            inp, lab, pos = inp.pin_memory(), lab.pin_memory(), pos.pin_memory()
        return {"input": inp, "positions": pos}, lab

    def __iter__(self):
        while True:
            batch = self._make(self.batch_idx)
            self.batch_idx += 1
            yield batch

    def state_dict(self):
        return {"version": 1, "dp_world_size": self.dp_world_size, f"dp_rank_{self.dp_rank}": {"batch_idx": self.batch_idx}}

    def load_state_dict(self, sd):
        if not sd:
            return
        if sd.get("dp_world_size", self.dp_world_size) != self.dp_world_size:
            raise ValueError(
                f"dataloader state was saved with dp degree {sd.get('dp_world_size')}, cannot resume with "
                f"{self.dp_world_size}"
            )
        key = f"dp_rank_{self.dp_rank}"
        if key in sd:
            self.batch_idx = int(sd[key]["batch_idx"])


class PrefetchIterator:
    """Background-thread prefetch of up to ``depth`` batches (parity: Grain's
    ``ThreadPrefetchIterDataset`` use in data/loader.py:61-178)."""

    _END = object()

    def __init__(self, it: Iterator, depth: int = 2):
        self._q: queue.Queue = queue.Queue(maxsize=max(1, depth))
        self._it = it
        self._err: BaseException | None = None
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        try:
            for item in self._it:
                while not self._stop.is_set():
                    try:
                        self._q.put(item, timeout=0.1)
                        break
                    except queue.Full:
                        continue
                if self._stop.is_set():
                    return
        except BaseException as e:  # surfaced on the consumer side
            self._err = e
        self._q.put(self._END)

    def __iter__(self):
        return self

    def __next__(self):
        item = self._q.get()
        if item is self._END:
            if self._err is not None:
                raise self._err
            raise StopIteration
        return item

    def close(self):
        self._stop.set()
