"""Single-turn math questions with a verifiable final answer (the task family of the reference's DAPO example).

The model is asked to end with ``Answer: <value>`` or ``\\boxed{<value>}``.  ``score_math_response`` extracts the
last such expression, normalises both sides (dollar signs, ``\\left`` / ``\\right``, spacing, thousands separators,
``\\frac{a}{b}`` and ``\\dfrac``, ``\\text{...}`` units, a trailing period, percent signs) and compares them as exact
rationals when both parse as numbers, as normalised strings otherwise.  The reward is binary.

Questions come from a JSONL file (``{"prompt": ..., "answer": ...}`` per line) or, without one, from a seeded
generator of integer-arithmetic problems, so the example runs offline.

Parity: torchtitan/experiments/rl/examples/dapo_math/{data.py:28-138, env.py:21-41, rubric.py:29-68} (the
reference checks equivalence with the Math-Verify package and reads the DAPO-Math-17k / AIME-2025 datasets).
"""

from __future__ import annotations

import json
import random
import re
from dataclasses import dataclass
from fractions import Fraction

from torchtitan_b200.config import Configurable

from ..environment import MessageEnv, MessageEnvInit, MessageEnvStep
from ..rollouter import RewardFn
from ..records import Message, Rollout

__all__ = ["MathSample", "MathDataset", "MathEnv", "RewardMathAnswer", "score_math_response", "extract_final_answer",
           "normalize_answer"]

_INSTRUCTION = ("Solve the problem step by step. The last line of your response must be 'Answer: $ANSWER' "
                "(without quotes) where $ANSWER is the final answer.\n\n")


@dataclass(frozen=True, kw_only=True, slots=True)
class MathSample:
    prompt: str
    ground_truth: str


class MathDataset(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        path: str | None = None
        seed: int = 0
        num_samples: int | None = None
        """Restart the stream after this many samples (a fixed evaluation set); None: endless."""

    def __init__(self, config: Config | None = None, **_):
        self.config = config or MathDataset.Config()
        self._rows = None
        if self.config.path:
            with open(self.config.path, encoding="utf-8") as f:
                self._rows = [json.loads(ln) for ln in f if ln.strip()]
            if not self._rows:
                raise ValueError(f"{self.config.path}: no samples")
        self._rng = random.Random(self.config.seed)
        self._n = 0

    def __iter__(self):
        return self

    def state_dict(self) -> dict:
        return {"rng_state": self._rng.getstate(), "n": self._n}

    def load_state_dict(self, state: dict) -> None:
        s = state["rng_state"]
        self._rng.setstate((s[0], tuple(s[1]), s[2]))
        self._n = state["n"]

    def __next__(self) -> MathSample:
        if self.config.num_samples and self._n >= self.config.num_samples:
            self._rng, self._n = random.Random(self.config.seed), 0
        self._n += 1
        if self._rows is not None:
            row = self._rows[self._rng.randrange(len(self._rows))]
            return MathSample(prompt=_INSTRUCTION + row["prompt"], ground_truth=str(row["answer"]))
        a, b, c = (self._rng.randint(2, 99) for _ in range(3))
        op = self._rng.choice(["+", "-", "*"])
        value = {"+": a + b, "-": a - b, "*": a * b}[op] * c
        return MathSample(prompt=f"{_INSTRUCTION}Compute ({a} {op} {b}) * {c}.", ground_truth=str(value))


class MathEnv(MessageEnv):
    @dataclass(kw_only=True, slots=True)
    class Config(MessageEnv.Config):
        pass

    def __init__(self, config: Config | None = None, *, env_input: MathSample):
        self.sample = env_input

    async def init(self) -> MessageEnvInit:
        return MessageEnvInit(init_prompt_messages=[{"role": "user", "content": self.sample.prompt}])

    async def step(self, completion_message: Message) -> MessageEnvStep:
        return MessageEnvStep(done=True)


def _last_boxed(text: str) -> str | None:
    at = text.rfind("\\boxed{")
    if at < 0:
        return None
    depth, start = 0, at + len("\\boxed{")
    for i in range(start, len(text)):
        if text[i] == "{":
            depth += 1
        elif text[i] == "}":
            if depth == 0:
                return text[start:i]
            depth -= 1
    return None          # unbalanced braces


def extract_final_answer(response: str) -> str | None:
    """The last ``Answer: ...`` line if there is one, else the last ``\\boxed{...}``."""
    lines = re.findall(r"(?im)^\s*\**answer\**\s*[:：]\s*(.+?)\s*$", response)
    if lines:
        inner = _last_boxed(lines[-1])
        return inner if inner is not None else lines[-1]
    return _last_boxed(response)


def normalize_answer(s: str) -> str:
    s = s.strip().strip("$").strip()
    s = re.sub(r"\\(left|right|!|,|;|:| )", "", s)
    s = re.sub(r"\\text\{[^{}]*\}", "", s)               # units
    s = re.sub(r"\\d?frac\{([^{}]+)\}\{([^{}]+)\}", r"(\1)/(\2)", s)
    s = s.replace("\\%", "").replace("%", "").replace("^\\circ", "").replace("\\$", "")
    s = re.sub(r"(?<=\d),(?=\d{3}\b)", "", s)            # thousands separators
    s = re.sub(r"\s+", "", s).rstrip(".")
    return s


def _as_number(s: str) -> Fraction | None:
    t = s.replace("(", "").replace(")", "")
    try:
        if "/" in t:
            a, b = t.split("/")
            return Fraction(a) / Fraction(b)
        return Fraction(t)
    except (ValueError, ZeroDivisionError):
        return None


def score_math_response(response: str, ground_truth: str) -> float:
    got = extract_final_answer(response)
    if got is None:
        return 0.0
    a, b = normalize_answer(got), normalize_answer(ground_truth)
    if not b:
        return 0.0
    x, y = _as_number(a), _as_number(b)
    if x is not None and y is not None:
        return float(x == y)
    return float(a == b)


class RewardMathAnswer(RewardFn):
    @dataclass(kw_only=True, slots=True)
    class Config(RewardFn.Config):
        pass

    async def __call__(self, rollout: Rollout, env_input: MathSample) -> float:
        if not rollout.turns:
            return 0.0
        msg = rollout.turns[-1].completion_message
        return score_math_response((msg or {}).get("content") or "", env_input.ground_truth)
