"""Open-domain question answering with a ``search`` tool: a multi-turn, tool-calling task.

Every assistant turn either calls ``search`` (the environment answers with a ``tool`` message holding the best
matching passages) or gives its final answer, which ends the rollout.  The reward is exact match of the normalised
answer against the golden answers, with two optional levers against answering from memory: a deduction for a correct
answer that never searched, and partial credit when a search surfaced a golden answer but the final answer is wrong.

Retrieval runs in process over a passage file (one ``title<TAB>text`` per line; scored by inverse-document-frequency
weighted term overlap) or, with ``search_url``, against an HTTP retrieval server (``{"queries": [...], "topk": k}``
-> ``{"result": [[{"contents": "title\\nbody"}, ...]]}``); a failed request yields an empty result instead of
failing the rollout.  Questions come from a JSONL file (``{"question": ..., "golden_answers": [...]}``).

Parity: torchtitan/experiments/rl/examples/search_r1/{data.py:19-119, env.py:58-169, rubric.py:26-127}.
"""

from __future__ import annotations

import asyncio
import json
import math
import random
import re
import string
from dataclasses import dataclass

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from ..environment import MessageEnv, MessageEnvInit, MessageEnvStep
from ..rollouter import RewardFn
from ..records import Message, Rollout

__all__ = ["SearchSample", "SearchDataset", "PassageIndex", "SearchEnv", "RewardExactMatch", "SEARCH_TOOL", "normalize_answer"]

SEARCH_TOOL = {
    "name": "search",
    "description": "Look up passages for a query. Use it whenever you need external facts to answer the question.",
    "parameters": {"type": "object", "properties": {"query": {"type": "string", "description": "The search query."}},
                   "required": ["query"]},
}
_INSTRUCTION = ("Answer the question. Use the search tool to look up any facts you are unsure of. When you know the "
                "answer, reply with only the answer itself, with no explanation.\n\nQuestion: ")


@dataclass(frozen=True, kw_only=True, slots=True)
class SearchSample:
    question: str
    golden_answers: tuple[str, ...]


class SearchDataset(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        path: str
        seed: int = 0

    def __init__(self, config: Config, **_):
        with open(config.path, encoding="utf-8") as f:
            self._rows = [json.loads(ln) for ln in f if ln.strip()]
        if not self._rows:
            raise ValueError(f"{config.path}: no questions")
        self._rng = random.Random(config.seed)

    def __iter__(self):
        return self

    def state_dict(self) -> dict:
        return {"rng_state": self._rng.getstate()}

    def load_state_dict(self, state: dict) -> None:
        s = state["rng_state"]
        self._rng.setstate((s[0], tuple(s[1]), s[2]))

    def __next__(self) -> SearchSample:
        row = self._rows[self._rng.randrange(len(self._rows))]
        gold = row["golden_answers"]
        return SearchSample(question=row["question"], golden_answers=tuple([gold] if isinstance(gold, str) else gold))


def _terms(text: str) -> list[str]:
    return re.findall(r"[a-z0-9]+", text.lower())


class PassageIndex:
    """Term-overlap retrieval with idf weights over ``(title, text)`` passages; enough for tests and small corpora."""

    def __init__(self, passages: list[tuple[str, str]]):
        self.passages = passages
        self._tf = [dict() for _ in passages]
        df: dict[str, int] = {}
        for i, (title, text) in enumerate(passages):
            for t in _terms(title + " " + text):
                self._tf[i][t] = self._tf[i].get(t, 0) + 1
            for t in self._tf[i]:
                df[t] = df.get(t, 0) + 1
        n = max(len(passages), 1)
        self._idf = {t: math.log(1 + n / c) for t, c in df.items()}

    @classmethod
    def from_file(cls, path: str) -> "PassageIndex":
        rows = []
        with open(path, encoding="utf-8") as f:
            for ln in f:
                if ln.strip():
                    title, _, text = ln.rstrip("\n").partition("\t")
                    rows.append((title, text))
        return cls(rows)

    def search(self, query: str, topk: int) -> list[dict]:
        q = set(_terms(query))
        scored = []
        for i, tf in enumerate(self._tf):
            s = sum(self._idf[t] * (1 + math.log(tf[t])) for t in q if t in tf)
            if s > 0:
                scored.append((s, -i))
        scored.sort(reverse=True)
        return [{"contents": f"{self.passages[-j][0]}\n{self.passages[-j][1]}"} for _, j in scored[:topk]]


def _format(docs: list[dict]) -> str:
    out = ""
    for i, d in enumerate(docs):
        title, _, body = (d.get("contents", "") if isinstance(d, dict) else "").partition("\n")
        out += f"Doc {i + 1}(Title: {title}) {body}\n"
    return out


_INDEXES: dict[str, PassageIndex] = {}


class SearchEnv(MessageEnv):
    @dataclass(kw_only=True, slots=True)
    class Config(MessageEnv.Config):
        passages_path: str | None = None
        search_url: str | None = None
        topk: int = 3
        timeout_s: float = 60.0

        def __post_init__(self):
            if (self.passages_path is None) == (self.search_url is None):
                raise ValueError("give exactly one of passages_path (in-process retrieval) and search_url")

    def __init__(self, config: Config, *, env_input: SearchSample):
        self.config, self.sample = config, env_input

    async def init(self) -> MessageEnvInit:
        return MessageEnvInit(init_prompt_messages=[{"role": "user", "content": _INSTRUCTION + self.sample.question}],
                              tools=[SEARCH_TOOL])

    async def _search(self, query: str) -> str:
        c = self.config
        if not query:
            return ""
        if c.passages_path is not None:
            if c.passages_path not in _INDEXES:
                _INDEXES[c.passages_path] = PassageIndex.from_file(c.passages_path)
            return _format(_INDEXES[c.passages_path].search(query, c.topk))
        try:
            import aiohttp

            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=c.timeout_s)) as session:
                async with session.post(c.search_url, json={"queries": [query], "topk": c.topk, "return_scores": False}) as r:
                    r.raise_for_status()
                    data = await r.json()
            return _format((data.get("result") or [[]])[0])
        except Exception as e:          # one flaky request must not fail the rollout
            logger.warning(f"search request to {c.search_url} failed: {e}")
            return ""

    async def step(self, completion_message: Message) -> MessageEnvStep:
        calls = completion_message.get("tool_calls") or []
        if not calls:
            return MessageEnvStep(done=True)
        queries = []
        for call in calls:
            args = call.get("arguments", {})
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except json.JSONDecodeError:
                    args = {}
            q = args.get("query", "") if isinstance(args, dict) else ""
            queries.append(q if isinstance(q, str) else "")
        found = await asyncio.gather(*(self._search(q) for q in queries))
        return MessageEnvStep(env_messages=[{"role": "tool", "content": p} for p in found])


def normalize_answer(s: str) -> str:
    s = "".join(ch for ch in s.lower() if ch not in set(string.punctuation))
    return " ".join(re.sub(r"\b(a|an|the)\b", " ", s).split())


class RewardExactMatch(RewardFn):
    @dataclass(kw_only=True, slots=True)
    class Config(RewardFn.Config):
        score: float = 1.0
        no_search_penalty: float = 0.0
        """Deducted from a correct answer that never called the tool."""
        retrieval_score: float = 0.0
        """Credit for a wrong or missing answer when a search result contained a golden answer."""

    async def __call__(self, rollout: Rollout, env_input: SearchSample) -> float:
        c = self.config
        gold = [normalize_answer(g) for g in env_input.golden_answers]
        last = (rollout.turns[-1].completion_message or {}) if rollout.turns else {}
        answer = None if last.get("tool_calls") else (last.get("content") or "").strip() or None
        searched = any((t.completion_message or {}).get("tool_calls") for t in rollout.turns)
        if answer is not None and normalize_answer(answer) in gold:
            return c.score if searched else c.score - c.no_search_penalty
        if c.retrieval_score:
            for t in rollout.turns:
                for msg in t.env_messages:
                    if msg.get("role") == "tool" and isinstance(msg.get("content"), str):
                        hay = f" {normalize_answer(msg['content'])} "
                        if any(f" {g} " in hay for g in gold):
                            return c.retrieval_score
        return 0.0
