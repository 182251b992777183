"""``SamplingParams`` with the reference's field names, defaults and validation
(kairyu/sampling_params.py:149-313).  Fields that belong to layers this engine
does not have (``n``/``best_of`` fan-out, stop strings, logprob reports,
structured output) are validated and then refused where they would matter."""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Sequence

_INT64_MAX = (1 << 63) - 1
_INT64_MIN = -(1 << 63)
_UINT64_MAX = (1 << 64) - 1


def _normalize_stop(stop: str | Sequence[str] | None) -> tuple[str, ...]:
    if stop is None:
        return ()
    if isinstance(stop, str):
        return (stop,)
    return tuple(stop)


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
        object.__setattr__(self, "stop", _normalize_stop(self.stop))
        object.__setattr__(self, "stop_token_ids", tuple(self.stop_token_ids) if self.stop_token_ids else ())
        self._validate()

    def _validate(self) -> None:
        if self.seed is not None and (type(self.seed) is not int or not _INT64_MIN <= self.seed <= _UINT64_MAX):
            raise ValueError("seed must fit signed or unsigned 64-bit range")
        if type(self.top_k) is not int or self.top_k > _INT64_MAX:
            raise ValueError("top_k must be a signed 64-bit integer")
        if any(type(t) is not int or not 0 <= t <= _INT64_MAX for t in self.stop_token_ids):
            raise ValueError("stop_token_ids must contain only non-negative 64-bit integers")
        if self.n < 1:
            raise ValueError(f"n must be >= 1, got {self.n}")
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError(f"top_k must be -1 or >= 1, got {self.top_k}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.repetition_penalty <= 0.0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError(f"presence_penalty must be in [-2, 2], got {self.presence_penalty}")
        if not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError(f"frequency_penalty must be in [-2, 2], got {self.frequency_penalty}")
        if self.max_tokens is not None and (type(self.max_tokens) is not int or not 1 <= self.max_tokens <= _INT64_MAX):
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")
        if type(self.min_tokens) is not int or not 0 <= self.min_tokens <= _INT64_MAX:
            raise ValueError(f"min_tokens must be >= 0, got {self.min_tokens}")
        if self.max_tokens is not None and self.min_tokens > self.max_tokens:
            raise ValueError(
                f"min_tokens must be <= max_tokens, got min_tokens={self.min_tokens}, max_tokens={self.max_tokens}"
            )
        for name in ("logprobs", "prompt_logprobs"):
            value = getattr(self, name)
            if value is not None and (type(value) is not int or not _INT64_MIN <= value <= _INT64_MAX):
                raise ValueError(f"{name} must be a signed 64-bit integer or None")

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
