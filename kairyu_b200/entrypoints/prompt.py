"""Prompt kinds (kairyu/engine/prompt.py:58-92): text, or caller-supplied token
ids, which bypass the tokenizer."""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from typing import Union

_MAX_TOKEN_ID = (1 << 64) - 1


@dataclass(frozen=True)
class TextPrompt:
    prompt: str


@dataclass(frozen=True)
class TokensPrompt:
    prompt_token_ids: tuple[int, ...]
    prompt: str | None = None

    def __post_init__(self) -> None:
        token_ids = self.prompt_token_ids
        if isinstance(token_ids, (str, bytes, bytearray)) or not isinstance(token_ids, Sequence):
            raise TypeError("TokensPrompt.prompt_token_ids must be a sequence of integers")
        copied = tuple(token_ids)
        if not copied:
            raise ValueError("TokensPrompt.prompt_token_ids must not be empty")
        for token_id in copied:
            if type(token_id) is not int:
                raise TypeError(
                    f"TokensPrompt.prompt_token_ids must contain integers, not {type(token_id).__name__}"
                )
            if not 0 <= token_id <= _MAX_TOKEN_ID:
                raise ValueError("TokensPrompt.prompt_token_ids values must be non-negative")
        if self.prompt is not None and type(self.prompt) is not str:
            raise TypeError("TokensPrompt.prompt must be a string or None")
        object.__setattr__(self, "prompt_token_ids", copied)


PromptInput = Union[str, TextPrompt, TokensPrompt, Mapping]


def normalize_prompt(prompt: object) -> TextPrompt | TokensPrompt:
    if isinstance(prompt, (TextPrompt, TokensPrompt)):
        return prompt
    if isinstance(prompt, str):
        return TextPrompt(prompt)
    if isinstance(prompt, Mapping):
        if "prompt_token_ids" in prompt:
            return TokensPrompt(tuple(prompt["prompt_token_ids"]), prompt.get("prompt"))
        if "prompt" in prompt:
            return TextPrompt(prompt["prompt"])
    raise TypeError(f"unsupported prompt type {type(prompt).__name__}")
