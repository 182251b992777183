"""``SamplingParams`` with the reference's field names, defaults and validation
(kairyu/sampling_params.py:149-313).  Fields that belong to layers this engine
does not have (``n``/``best_of`` fan-out, stop strings, logprob reports,
structured output) are validated and then refused where they would matter."""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Sequence

I64_LOW, I64_HIGH, U64_HIGH = -(2**63), 2**63 - 1, 2**64 - 1


def _is_int(value: object) -> bool:
    return type(value) is int  # bool is not accepted as an integer


@dataclass(frozen=True)
class SamplingParams:
    n: int = 1
    best_of: int | None = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    seed: int | None = None
    stop: str | Sequence[str] | None = None
    stop_token_ids: Sequence[int] | None = None
    max_tokens: int | None = 16
    min_tokens: int = 0
    logprobs: int | None = None
    prompt_logprobs: int | None = None
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    extra_args: dict = field(default_factory=dict, compare=False)

    def __post_init__(self) -> None:
        stop = self.stop
        stop = () if stop is None else (stop,) if isinstance(stop, str) else tuple(stop)
        object.__setattr__(self, "stop", stop)
        object.__setattr__(self, "stop_token_ids", tuple(self.stop_token_ids or ()))
        problems = self._problems()
        if problems:
            raise ValueError("; ".join(problems))

    def _problems(self) -> list[str]:
        """Everything wrong with the values, in words; empty when they are fine.  The rules are the
        reference's (kairyu/sampling_params.py:222-313): integers are true ints within 64 bits, the
        filters' ranges, min_tokens within max_tokens."""
        found: list[str] = []

        def integer(name: str, low: int, high: int, *, optional: bool = False) -> bool:
            value = getattr(self, name)
            if value is None and optional:
                return False
            if not _is_int(value) or not low <= value <= high:
                found.append(f"{name}={value!r} is not an integer in [{low}, {high}]")
                return False
            return True

        def real(name: str, ok: bool, rule: str) -> None:
            if not ok:
                found.append(f"{name}={getattr(self, name)!r} must be {rule}")

        integer("seed", I64_LOW, U64_HIGH, optional=True)
        integer("logprobs", I64_LOW, I64_HIGH, optional=True)
        integer("prompt_logprobs", I64_LOW, I64_HIGH, optional=True)
        if integer("top_k", -1, I64_HIGH) and self.top_k == 0:
            found.append("top_k=0 keeps no token; use -1 for no limit or a count >= 1")
        integer("n", 1, I64_HIGH)
        has_max = integer("max_tokens", 1, I64_HIGH, optional=True)
        if integer("min_tokens", 0, I64_HIGH) and has_max and self.min_tokens > self.max_tokens:
            found.append(f"min_tokens={self.min_tokens} exceeds max_tokens={self.max_tokens}")
        if not all(_is_int(token) and 0 <= token <= I64_HIGH for token in self.stop_token_ids):
            found.append("stop_token_ids holds something that is not a token id (an integer in [0, 2^63))")
        real("temperature", self.temperature >= 0.0, "0 (greedy) or positive")
        real("top_p", 0.0 < self.top_p <= 1.0, "in (0, 1]")
        real("min_p", 0.0 <= self.min_p <= 1.0, "in [0, 1]")
        real("repetition_penalty", self.repetition_penalty > 0.0, "positive")
        real("presence_penalty", -2.0 <= self.presence_penalty <= 2.0, "in [-2, 2]")
        real("frequency_penalty", -2.0 <= self.frequency_penalty <= 2.0, "in [-2, 2]")
        return found

    def clone(self, **overrides: object) -> "SamplingParams":
        return dataclasses.replace(self, **overrides)  # type: ignore[arg-type]

    @property
    def is_greedy_pure(self) -> bool:
        """Argmax with no penalties (kairyu/engine/core/sampling_types.py:61-70)."""
        return (
            self.temperature == 0.0
            and self.presence_penalty == 0.0
            and self.frequency_penalty == 0.0
            and self.repetition_penalty == 1.0
        )
