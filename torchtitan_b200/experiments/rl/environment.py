"""Environments.  A user writes a ``MessageEnv`` (``init`` gives the opening messages and tool specs, ``step``
answers an assistant message and says when the episode is done); ``TokenEnv`` wraps it for the rollout loop, which
works in tokens: it renders prompts, parses completions and turns every way an episode can end early (completion
cut by the length limit, aborted request, unparsable completion, environment step over its time limit, prompt
beyond the token budget, turn cap) into a terminal ``RolloutStatus`` instead of an exception.

Parity: torchtitan/experiments/rl/environment/message.py:18-108, environment/token.py:24-301.
"""

from __future__ import annotations

import abc
import asyncio
from dataclasses import dataclass, field
from typing import Any

from torchtitan_b200.config import Configurable
from torchtitan_b200.utils.logging import logger

from .records import Completion, Message, RolloutStatus

__all__ = ["MessageEnvInit", "MessageEnvStep", "MessageEnv", "TokenEnvOutput", "TokenEnv"]


@dataclass(kw_only=True, slots=True)
class MessageEnvInit:
    init_prompt_messages: list[Message]
    tools: list[dict[str, Any]] = field(default_factory=list)


@dataclass(kw_only=True, slots=True)
class MessageEnvStep:
    env_messages: list[Message] = field(default_factory=list)   # tool / user replies; never assistant messages
    done: bool = False
    env_rewards: dict[str, float] = field(default_factory=dict)

    def __post_init__(self):
        if any(m.get("role") == "assistant" for m in self.env_messages):
            raise ValueError("an environment's reply may not contain assistant messages")


class MessageEnv(Configurable, abc.ABC):
    """Static parameters live in ``Config``; the per-episode dataset sample comes through
    ``Config.build(env_input=sample)``.  One instance serves one rollout."""

    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    @abc.abstractmethod
    async def init(self) -> MessageEnvInit: ...

    @abc.abstractmethod
    async def step(self, completion_message: Message) -> MessageEnvStep: ...

    async def close(self) -> None:
        return None


@dataclass(kw_only=True, slots=True)
class TokenEnvOutput:
    status: RolloutStatus
    next_prompt_token_ids: list[int] | None = None     # None once the episode is over
    next_prompt_messages: list[Message] | None = None
    completion_message: Message | None = None          # None on init and on a parse error
    env_messages: list[Message] = field(default_factory=list)
    env_rewards: dict[str, float] = field(default_factory=dict)


class TokenEnv(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        max_rollout_tokens: int | None = None
        """A next prompt of this many tokens or more ends the episode (``truncated_prompt_too_long``)."""
        step_timeout_s: float | None = 1800.0
        max_num_turns: int | None = None

    def __init__(self, config: Config | None = None, *, message_env: MessageEnv, renderer):
        self.config = config or TokenEnv.Config()
        self._env, self._renderer = message_env, renderer
        self._messages: list[Message] = []
        self._tools = None
        self._last_prompt: list[int] = []
        self._turns = 0

    def _too_long(self, n: int) -> bool:
        cap = self.config.max_rollout_tokens
        return cap is not None and n >= cap

    async def init(self) -> TokenEnvOutput:
        first = await self._env.init()
        self._messages = list(first.init_prompt_messages)
        self._tools = first.tools or None
        ids = await asyncio.to_thread(self._renderer.render_ids, messages=self._messages, tools=self._tools,
                                      add_generation_prompt=True)
        if self._too_long(len(ids)):
            return TokenEnvOutput(status=RolloutStatus.TRUNCATED_PROMPT_TOO_LONG, next_prompt_token_ids=ids,
                                  next_prompt_messages=self._messages)
        self._last_prompt = ids
        return TokenEnvOutput(status=RolloutStatus.ONGOING, next_prompt_token_ids=ids, next_prompt_messages=self._messages)

    async def step(self, completion: Completion) -> TokenEnvOutput:
        self._turns += 1
        try:
            parsed = await asyncio.to_thread(self._renderer.parse_response, token_ids=completion.token_ids)
        except Exception as e:
            logger.warning(f"completion of {len(completion.token_ids)} tokens did not parse ({e}): error_parse")
            return TokenEnvOutput(status=RolloutStatus.ERROR_PARSE)
        message: Message = {"role": "assistant", "content": parsed.content}
        if parsed.reasoning_content:
            message["reasoning_content"] = parsed.reasoning_content
        if parsed.tool_calls:
            message["tool_calls"] = parsed.tool_calls
        if completion.finish_reason == "length":
            return TokenEnvOutput(status=RolloutStatus.TRUNCATED_LENGTH, completion_message=message)
        if completion.finish_reason == "abort":
            return TokenEnvOutput(status=RolloutStatus.ERROR_ABORT, completion_message=message)
        try:
            reply = await asyncio.wait_for(self._env.step(message), timeout=self.config.step_timeout_s)
        except (asyncio.TimeoutError, TimeoutError):
            logger.warning(f"environment step exceeded {self.config.step_timeout_s} s: error_timeout")
            return TokenEnvOutput(status=RolloutStatus.ERROR_TIMEOUT, completion_message=message)
        self._messages = self._messages + [message] + reply.env_messages
        ended = dict(completion_message=message, env_messages=reply.env_messages, env_rewards=reply.env_rewards)
        if reply.done:
            return TokenEnvOutput(status=RolloutStatus.COMPLETED, **ended)
        if self.config.max_num_turns is not None and self._turns >= self.config.max_num_turns:
            return TokenEnvOutput(status=RolloutStatus.TRUNCATED_MAX_TURNS, **ended)
        bridged = await asyncio.to_thread(self._renderer.bridge_to_next_turn, previous_prompt_ids=self._last_prompt,
                                          previous_completion_ids=completion.token_ids,
                                          new_messages=reply.env_messages, tools=self._tools)
        if bridged is None:
            ids = await asyncio.to_thread(self._renderer.render_ids, messages=self._messages, tools=self._tools,
                                          add_generation_prompt=True)
        else:
            ids = bridged.token_ids
        if self._too_long(len(ids)):
            return TokenEnvOutput(status=RolloutStatus.TRUNCATED_PROMPT_TOO_LONG, **ended)
        self._last_prompt = ids
        return TokenEnvOutput(status=RolloutStatus.ONGOING, next_prompt_token_ids=ids, next_prompt_messages=self._messages,
                              **ended)

    async def close(self) -> None:
        await self._env.close()
