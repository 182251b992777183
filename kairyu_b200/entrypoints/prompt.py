"""Prompt kinds (kairyu/engine/prompt.py:58-92): text, or caller-supplied token
ids, which bypass the tokenizer."""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from typing import Union

@dataclass(frozen=True)
class TextPrompt:
    prompt: str


@dataclass(frozen=True)
class TokensPrompt:
    """Token ids given by the caller; ``prompt`` may carry the text they came from.  The ids are
    kept as a tuple of true ints in [0, 2^64); anything else is refused at construction
    (kairyu/engine/prompt.py:58-92 has the same rules)."""

    prompt_token_ids: tuple[int, ...]
    prompt: str | None = None

    def __post_init__(self) -> None:
        given = self.prompt_token_ids
        if isinstance(given, (str, bytes, bytearray)) or not isinstance(given, Sequence):
            raise TypeError(f"prompt_token_ids: a sequence of token ids is needed, got {type(given).__name__}")
        ids = tuple(given)
        strangers = sorted({type(item).__name__ for item in ids if type(item) is not int})
        if strangers:
            raise TypeError(f"prompt_token_ids: token ids are integers; found {', '.join(strangers)}")
        if not ids:
            raise ValueError("prompt_token_ids: at least one token is needed")
        if min(ids) < 0 or max(ids) >= 2**64:
            raise ValueError("prompt_token_ids: token ids lie in [0, 2^64)")
        if not (self.prompt is None or type(self.prompt) is str):
            raise TypeError("prompt: the text of a TokensPrompt is a str or None")
        object.__setattr__(self, "prompt_token_ids", ids)


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
