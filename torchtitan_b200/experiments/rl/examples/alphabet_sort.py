"""Multi-turn alphabetical sorting: the task of the reference's main RL example, self-contained.

A sample shows a few CamelCase names and asks for them sorted (by first or by last name) inside an
``<alphabetical_sorted>`` block; every further turn adds names and asks for the whole list re-sorted inside
``<combined_alphabetical_sorted>``, new entries marked ``// new name!``.  The reward is the similarity of the
answered list to the expected one (difflib ratio over the lower-cased lines, raised to a power so that only
near-perfect orderings score near 1), averaged over the expected turns: a rollout that ends early scores 0 for the
turns it never reached.

Names come from ``names_path`` (one ``First Last`` per line) or, without it, from a pool synthesised from
syllables with the dataset seed: no download is needed.

Parity: torchtitan/experiments/rl/examples/alphabet_sort/{data.py:19-185, env.py:21-80, rubric.py:19-116,
rollouter.py:20-62} (the reference draws names from a Hugging Face dataset of arXiv authors).
"""

from __future__ import annotations

import difflib
import random
import re
from dataclasses import dataclass
from typing import Sequence

from torchtitan_b200.config import Configurable

from ..environment import MessageEnv, MessageEnvInit, MessageEnvStep
from ..rollouter import RewardFn
from ..records import Message, Rollout

__all__ = ["AlphabetSortSample", "AlphabetSortDataset", "AlphabetSortEnv", "RewardAlphabetSort", "score_sorted_list"]

_SYLLABLES = ("an", "bel", "cor", "dan", "el", "fen", "gar", "hal", "ing", "jor", "kel", "lin", "mar", "nor", "ol",
              "per", "quin", "ros", "sten", "tor", "ul", "van", "wen", "xan", "yor", "zel")


@dataclass(frozen=True, slots=True)
class _Author:
    display: str      # "MarcChardin"
    first: str
    last: str


@dataclass(frozen=True, kw_only=True, slots=True)
class AlphabetSortSample:
    new_names_per_turn: tuple[tuple[str, ...], ...]     # [turn][names shown at that turn]
    expected_names: tuple[tuple[str, ...], ...]         # [turn][the whole list so far, sorted]
    sort_by_first_name: bool


def _synthetic_pool(seed: int, n: int = 2000) -> tuple[_Author, ...]:
    rng = random.Random(seed ^ 0x5EED)
    seen, out = set(), []
    while len(out) < n:
        first = "".join(rng.sample(_SYLLABLES, rng.randint(1, 2))).capitalize()
        last = "".join(rng.sample(_SYLLABLES, rng.randint(2, 3))).capitalize()
        if first + last not in seen:
            seen.add(first + last)
            out.append(_Author(first + last, first.lower(), last.lower()))
    return tuple(out)


def _pool_from_file(path: str) -> tuple[_Author, ...]:
    seen, out = set(), []
    with open(path, encoding="utf-8") as f:
        for line in f:
            parts = line.split()
            if len(parts) == 2 and "".join(parts) not in seen:      # names of exactly two words
                seen.add("".join(parts))
                out.append(_Author("".join(parts), parts[0].lower(), parts[1].lower()))
    return tuple(out)


class AlphabetSortDataset(Configurable):
    """An endless, seeded stream of samples; ``state_dict`` / ``load_state_dict`` resume it exactly."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        seed: int = 1337420
        max_turns: int = 3
        max_names_per_turn: int = 5
        names_path: str | None = None

        def __post_init__(self):
            if self.max_turns < 1 or self.max_names_per_turn < 1:
                raise ValueError(f"max_turns and max_names_per_turn must be >= 1, got {self.max_turns}, {self.max_names_per_turn}")

    def __init__(self, config: Config | None = None, **_):
        self.config = config or AlphabetSortDataset.Config()
        c = self.config
        self._pool = _pool_from_file(c.names_path) if c.names_path else _synthetic_pool(c.seed)
        self._rng = random.Random(c.seed)

    def __iter__(self):
        return self

    def state_dict(self) -> dict:
        return {"rng_state": self._rng.getstate()}

    def load_state_dict(self, state: dict) -> None:
        s = state["rng_state"]
        self._rng.setstate((s[0], tuple(s[1]), s[2]))         # a checkpoint round trip turns the tuple into a list

    def __next__(self) -> AlphabetSortSample:
        c, rng = self.config, self._rng
        counts = [rng.randint(1, c.max_names_per_turn) for _ in range(rng.randint(1, c.max_turns))]
        drawn = rng.sample(self._pool, k=sum(counts))
        by_first = rng.choice([True, False])
        key = (lambda a: (a.first, a.last)) if by_first else (lambda a: (a.last, a.first))
        shown, expected, seen, at = [], [], [], 0
        for turn, n in enumerate(counts):
            new = drawn[at:at + n]
            at += n
            seen += new
            names = [a.display for a in new]
            rng.shuffle(names)
            shown.append(tuple(names))
            fresh = set(new) if turn else set()
            expected.append(tuple(a.display + (" // new name!" if a in fresh else "") for a in sorted(seen, key=key)))
        return AlphabetSortSample(new_names_per_turn=tuple(shown), expected_names=tuple(expected), sort_by_first_name=by_first)


class AlphabetSortEnv(MessageEnv):
    @dataclass(kw_only=True, slots=True)
    class Config(MessageEnv.Config):
        pass

    def __init__(self, config: Config | None = None, *, env_input: AlphabetSortSample):
        self.sample = env_input
        self._turn = 0

    def _ask(self, turn: int) -> str:
        s = self.sample
        names = "\n".join(s.new_names_per_turn[turn])
        by = "first" if s.sort_by_first_name else "last"
        if turn == 0:
            return (f"Sort these names alphabetically by {by} name, one per line, inside "
                    f"<alphabetical_sorted> and </alphabetical_sorted>:\n{names}")
        return (f"Add these names and give the whole list again, sorted by {by} name, inside "
                f"<combined_alphabetical_sorted> and </combined_alphabetical_sorted>; mark every name that is new in "
                f"this message with ' // new name!':\n{names}")

    async def init(self) -> MessageEnvInit:
        return MessageEnvInit(init_prompt_messages=[{"role": "user", "content": self._ask(0)}])

    async def step(self, completion_message: Message) -> MessageEnvStep:
        self._turn += 1
        if self._turn >= len(self.sample.new_names_per_turn):
            return MessageEnvStep(done=True)
        return MessageEnvStep(env_messages=[{"role": "user", "content": self._ask(self._turn)}])


def _answer_lines(text: str, tag: str) -> list[str]:
    blocks = re.findall(rf"<\s*{tag}\s*>(.*?)</\s*{tag}\s*>", text, re.S | re.I)
    return [ln.strip() for ln in blocks[-1].splitlines() if ln.strip()] if blocks else []


def score_sorted_list(response_text: str, *, expected_names: Sequence[str], xml_tag: str, similarity_power: int = 4) -> float:
    """In [0, 1]; 0 without an answer block; the LAST block counts when there are several."""
    got = _answer_lines(response_text, xml_tag)
    if not got:
        return 0.0
    a, b = "\n".join(x.lower() for x in got), "\n".join(x.lower() for x in expected_names)
    return difflib.SequenceMatcher(None, a, b).ratio() ** similarity_power


class RewardAlphabetSort(RewardFn):
    @dataclass(kw_only=True, slots=True)
    class Config(RewardFn.Config):
        similarity_power: int = 4

        def __post_init__(self):
            if self.similarity_power <= 0:
                raise ValueError(f"similarity_power must be positive, got {self.similarity_power}")

    async def __call__(self, rollout: Rollout, env_input: AlphabetSortSample) -> float:
        want = env_input.expected_names
        if not want:
            return 0.0
        total = 0.0
        for i, (turn, names) in enumerate(zip(rollout.turns, want)):
            text = (turn.completion_message or {}).get("content") or ""
            total += score_sorted_list(text, expected_names=names, similarity_power=self.config.similarity_power,
                                       xml_tag="alphabetical_sorted" if i == 0 else "combined_alphabetical_sorted")
        return total / len(want)
