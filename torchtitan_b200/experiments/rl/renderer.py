"""Chat messages <-> token ids for rollouts, on the framework's own tokenizers.

``ChatRenderer.render_ids`` turns a conversation into the prompt tokens of the next assistant turn: through the
tokenizer's Jinja chat template when it has one, otherwise through a ChatML layout
(``<|im_start|>role\\ncontent<|im_end|>\\n``).  ``parse_response`` decodes a sampled completion into content,
``<think>...</think>`` reasoning and ``<tool_call>{json}</tool_call>`` tool calls (the Hermes / Qwen convention;
malformed JSON raises, which the token environment records as a parse error).  ``bridge_to_next_turn`` extends the
previous prompt and completion *as tokens* with the environment's reply, so that the history of a multi-turn rollout
is never re-tokenised and the packed training sample stays a single growing prefix.

Parity: torchtitan/experiments/rl/renderer.py:32-93 (the reference wraps the external ``renderers`` package; its
three calls used by the token environment are the three methods here).
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any

from torchtitan_b200.config import Configurable

from .records import Message

__all__ = ["ChatRenderer", "ParsedResponse", "BridgedPrompt"]

_THINK = re.compile(r"<think>(.*?)</think>", re.S)
_TOOL = re.compile(r"<tool_call>(.*?)</tool_call>", re.S)


@dataclass(kw_only=True, slots=True)
class ParsedResponse:
    content: str
    reasoning_content: str | None = None
    tool_calls: list[dict[str, Any]] = field(default_factory=list)


@dataclass(kw_only=True, slots=True)
class BridgedPrompt:
    token_ids: list[int]


class ChatRenderer(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        use_chat_template: bool = True
        """Use the tokenizer's own chat template when it has one."""
        enable_thinking: bool = True
        """Keep ``<think>`` blocks as ``reasoning_content``; off: they are dropped from the parsed message."""
        preserve_all_thinking: bool = True
        """Keep earlier turns' reasoning in later prompts.  Off: history is re-rendered without it, the prefix of
        the next prompt changes and the rollout packs into several training samples."""
        turn_start: str = "<|im_start|>"
        turn_end: str = "<|im_end|>"

    def __init__(self, config: Config | None = None, *, tokenizer):
        self.config = config or ChatRenderer.Config()
        self.tokenizer = tokenizer
        self._end_ids = self._encode(self.config.turn_end)

    # -- text <-> ids ----------------------------------------------------------------------------------------------
    def _encode(self, text: str) -> list[int]:
        return list(self.tokenizer.encode(text, add_bos=False, add_eos=False))

    @property
    def eos_token_id(self) -> int:
        return int(self.tokenizer.eos_id)

    @property
    def stop_sequences(self) -> list[list[int]]:
        """Token sequences that end an assistant turn (besides EOS)."""
        return [self._end_ids] if self._end_ids else []

    def _message_text(self, m: Message) -> str:
        body = m.get("content") or ""
        if m.get("reasoning_content") and self.config.preserve_all_thinking:
            body = f"<think>{m['reasoning_content']}</think>{body}"
        for call in m.get("tool_calls") or []:
            body += f"<tool_call>{json.dumps(call, sort_keys=True)}</tool_call>"
        return f"{self.config.turn_start}{m['role']}\n{body}{self.config.turn_end}\n"

    def _tools_text(self, tools) -> str:
        if not tools:
            return ""
        specs = "\n".join(json.dumps(t, sort_keys=True) for t in tools)
        return (f"{self.config.turn_start}system\nYou may call these tools by writing "
                f"<tool_call>{{\"name\": ..., \"arguments\": {{...}}}}</tool_call>:\n{specs}{self.config.turn_end}\n")

    def render_ids(self, *, messages: list[Message], tools=None, add_generation_prompt: bool = True) -> list[int]:
        tok = self.tokenizer
        if self.config.use_chat_template and getattr(tok, "chat_template", None):
            text = tok.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tools=tools)
            return self._encode(text)
        text = self._tools_text(tools) + "".join(self._message_text(m) for m in messages)
        if add_generation_prompt:
            text += f"{self.config.turn_start}assistant\n"
        ids = self._encode(text)
        return ([int(tok.bos_id)] if getattr(tok, "bos_id", None) is not None else []) + ids

    def parse_response(self, *, token_ids: list[int]) -> ParsedResponse:
        ids = list(token_ids)
        while ids and ids[-1] == self.eos_token_id:
            ids.pop()
        text = self.tokenizer.decode(ids)
        if text.endswith(self.config.turn_end):
            text = text[:-len(self.config.turn_end)]
        reasoning = None
        found = _THINK.findall(text)
        if found:
            reasoning = "\n".join(s.strip() for s in found) if self.config.enable_thinking else None
            text = _THINK.sub("", text)
        calls = []
        for raw in _TOOL.findall(text):
            call = json.loads(raw)        # malformed JSON: ValueError -> the caller's parse-error path
            if not isinstance(call, dict) or "name" not in call:
                raise ValueError(f"tool call without a name: {raw!r}")
            calls.append(call)
        if "<tool_call>" in _TOOL.sub("", text):
            raise ValueError("unterminated <tool_call> block")
        return ParsedResponse(content=_TOOL.sub("", text).strip(), reasoning_content=reasoning, tool_calls=calls)

    def bridge_to_next_turn(self, *, previous_prompt_ids: list[int], previous_completion_ids: list[int],
                            new_messages: list[Message], tools=None) -> BridgedPrompt | None:
        """``previous prompt + completion`` kept token for token, then the closing of the assistant turn (if the
        sampler stopped on EOS or length rather than on the end marker), the new messages and the next generation
        prompt.  ``None`` when the history cannot be kept (reasoning is stripped from history, or the tokenizer's
        own template decides the layout): the caller re-renders from messages."""
        if not self.config.preserve_all_thinking:
            return None
        if self.config.use_chat_template and getattr(self.tokenizer, "chat_template", None):
            return None
        done = list(previous_completion_ids)      # verbatim, a trailing EOS included: the next prompt must extend it
        n = len(self._end_ids)
        closed = n > 0 and done[-n:] == self._end_ids
        tail = ("" if closed else self.config.turn_end) + "\n" + "".join(self._message_text(m) for m in new_messages)
        tail += f"{self.config.turn_start}assistant\n"
        return BridgedPrompt(token_ids=list(previous_prompt_ids) + done + self._encode(tail))
