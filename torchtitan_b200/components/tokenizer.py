"""Tokenizers.

``HuggingFaceTokenizer`` loads ``tokenizer.json`` (or ``vocab.json`` + ``merges.txt`` /
``vocab.txt``) from a folder with the ``tokenizers`` library, reads BOS/EOS from
``tokenizer_config.json`` / ``config.json`` / ``generation_config.json`` and finds
out whether the underlying pipeline already adds them, so that
``encode(text, add_bos, add_eos)`` never doubles a special token.  Chat templates are
rendered with jinja2.  Parity: torchtitan/components/tokenizer.py:19-550.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

__all__ = ["BaseTokenizer", "HuggingFaceTokenizer", "MultiModalTokenizer", "ByteTokenizer"]


class BaseTokenizer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    def __init__(self, config=None, **_):
        self.config = config
        self.eos_id = 0
        self.bos_id = None
        self.chat_template: str | None = None

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> list[int]:
        raise NotImplementedError

    def decode(self, ids: list[int], **kw) -> str:
        raise NotImplementedError

    def get_vocab_size(self) -> int:
        raise NotImplementedError

    def apply_chat_template(self, messages: list[dict[str, str]], add_generation_prompt: bool = False, **kw) -> str:
        if not self.chat_template:
            raise ValueError("this tokenizer has no chat template")
        import jinja2

        env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = lambda m: (_ for _ in ()).throw(ValueError(m))
        return env.from_string(self.chat_template).render(
            messages=messages, add_generation_prompt=add_generation_prompt,
            bos_token=getattr(self, "bos_token", "") or "", eos_token=getattr(self, "eos_token", "") or "", **kw)


class ByteTokenizer(BaseTokenizer):
    """UTF-8 bytes + BOS/EOS; used by tests and as a fallback when no tokenizer files exist."""

    def __init__(self, config=None, **_):
        super().__init__(config)
        self.bos_id, self.eos_id = 256, 257

    def encode(self, text, add_bos=True, add_eos=True):
        ids = list(text.encode("utf-8"))
        return ([self.bos_id] if add_bos else []) + ids + ([self.eos_id] if add_eos else [])

    def decode(self, ids, **kw):
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")

    def get_vocab_size(self):
        return 258


def _read_json(path: str) -> dict:
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


def _token_str(v: Any) -> str | None:
    if isinstance(v, dict):
        return v.get("content")
    return v if isinstance(v, str) else None


class HuggingFaceTokenizer(BaseTokenizer):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseTokenizer.Config):
        pass

    def __init__(self, config=None, *, tokenizer_path: str, **_):
        super().__init__(config)
        from tokenizers import Tokenizer

        self.tokenizer_path = tokenizer_path
        tj = os.path.join(tokenizer_path, "tokenizer.json")
        if os.path.exists(tj):
            self.tokenizer = Tokenizer.from_file(tj)
        else:
            self.tokenizer = self._from_vocab_files(tokenizer_path)
        cfg = _read_json(os.path.join(tokenizer_path, "tokenizer_config.json"))
        model_cfg = _read_json(os.path.join(tokenizer_path, "config.json"))
        gen_cfg = _read_json(os.path.join(tokenizer_path, "generation_config.json"))
        self.chat_template = cfg.get("chat_template")
        tmpl_file = os.path.join(tokenizer_path, "chat_template.jinja")
        if self.chat_template is None and os.path.exists(tmpl_file):
            with open(tmpl_file) as f:
                self.chat_template = f.read()
        self.bos_token = _token_str(cfg.get("bos_token"))
        self.eos_token = _token_str(cfg.get("eos_token"))
        self.bos_id = self.tokenizer.token_to_id(self.bos_token) if self.bos_token else None
        self.eos_id = self.tokenizer.token_to_id(self.eos_token) if self.eos_token else None
        for key, attr in (("bos_token_id", "bos_id"), ("eos_token_id", "eos_id")):
            if getattr(self, attr) is None:
                for src in (model_cfg, gen_cfg):
                    v = src.get(key)
                    if isinstance(v, list):
                        v = v[0] if v else None
                    if v is not None:
                        setattr(self, attr, int(v))
                        break
        self.hf_adds_bos, self.hf_adds_eos = self._probe_special_tokens()
        if self.eos_id is None:
            logger.warning("tokenizer has no EOS token; documents will not be separated by EOS")

    @staticmethod
    def _from_vocab_files(path: str):
        from tokenizers import Tokenizer, models, pre_tokenizers, decoders

        vocab_json, merges = os.path.join(path, "vocab.json"), os.path.join(path, "merges.txt")
        vocab_txt = os.path.join(path, "vocab.txt")
        if os.path.exists(vocab_json) and os.path.exists(merges):
            tok = Tokenizer(models.BPE.from_file(vocab_json, merges))
            tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            tok.decoder = decoders.ByteLevel()
            return tok
        if os.path.exists(vocab_json):
            with open(vocab_json) as f:
                vocab = json.load(f)
            return Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
        if os.path.exists(vocab_txt):
            with open(vocab_txt) as f:
                vocab = {line.rstrip("\n"): i for i, line in enumerate(f)}
            tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
            tok.pre_tokenizer = pre_tokenizers.Whitespace()
            return tok
        raise FileNotFoundError(
            f"no tokenizer files in '{path}' (expected tokenizer.json, or vocab.json + merges.txt, or vocab.txt)")

    def _probe_special_tokens(self) -> tuple[bool, bool]:
        ids = self.tokenizer.encode("a", add_special_tokens=True).ids
        adds_bos = self.bos_id is not None and len(ids) > 0 and ids[0] == self.bos_id
        adds_eos = self.eos_id is not None and len(ids) > 0 and ids[-1] == self.eos_id
        return adds_bos, adds_eos

    def encode(self, text, add_bos=True, add_eos=True):
        ids = self.tokenizer.encode(text, add_special_tokens=True).ids
        if add_bos and not self.hf_adds_bos and self.bos_id is not None:
            ids = [self.bos_id] + ids
        if not add_bos and self.hf_adds_bos and ids and ids[0] == self.bos_id:
            ids = ids[1:]
        if add_eos and not self.hf_adds_eos and self.eos_id is not None:
            ids = ids + [self.eos_id]
        if not add_eos and self.hf_adds_eos and ids and ids[-1] == self.eos_id:
            ids = ids[:-1]
        return ids

    def decode(self, ids, skip_special_tokens: bool = True, **kw):
        return self.tokenizer.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def get_vocab_size(self):
        return self.tokenizer.get_vocab_size(with_added_tokens=True)

    def token_to_id(self, tok: str):
        return self.tokenizer.token_to_id(tok)

    def id_to_token(self, i: int):
        return self.tokenizer.id_to_token(i)


class MultiModalTokenizer(HuggingFaceTokenizer):
    @dataclass(kw_only=True, slots=True)
    class Config(HuggingFaceTokenizer.Config):
        image_token: str = "<|image|>"
        video_token: str = "<|video|>"
        vision_start_token: str = "<|vision_start|>"
        vision_end_token: str = "<|vision_end|>"
        pad_token: str = "<|pad|>"

    def __init__(self, config, *, tokenizer_path: str, **kw):
        super().__init__(config, tokenizer_path=tokenizer_path, **kw)
        for name in ("image", "video", "vision_start", "vision_end", "pad"):
            tok = getattr(config, f"{name}_token")
            tid = self.tokenizer.token_to_id(tok)
            if tid is None:
                raise ValueError(f"special token {tok!r} is not in the vocabulary")
            setattr(self, f"{name}_id", tid)
