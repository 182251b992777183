"""Engine options, named as the reference's ``build_engine_loop`` names them
(kairyu/engine/kairyu_backend.py:467-500)."""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any

_DTYPES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "float": "float32",
}


def normalize_dtype(name: str, *, stored: str | None = None) -> str:
    """``auto`` follows the reference: bfloat16 on the GPU (kairyu_backend.py:974-980)."""
    if name == "auto":
        return "bfloat16"
    if name not in _DTYPES:
        raise ValueError(f"dtype must be one of auto, bfloat16, float32; got {name!r}")
    return _DTYPES[name]


@dataclass(frozen=True)
class EngineConfig:
    """Knobs of one engine instance.

    ``num_pages=None`` sizes the pool from ``gpu_memory_utilization``; an
    integer fixes it (page 0 is kept as the padding target of graph replays
    and is never handed to a request).
    """

    dtype: str = "bfloat16"
    device: str = "cuda"
    num_pages: int | None = None
    page_size: int = 16
    max_num_batched_tokens: int = 2048
    max_num_partial_prefills: int = 2
    max_num_seqs: int = 256
    max_model_len: int | None = None
    prefill_chunk_size: int | None = None
    gpu_memory_utilization: float = 0.9
    decode_mode: str | None = None  # None -> "cuda_graph" on CUDA, "eager" elsewhere
    cuda_graph_max_batch: int | None = None
    # capture steps that hold prompt portions once their shape has come twice (None: where decode graphs are on)
    portion_graphs: bool | None = None
    # Steps that may be launched before the oldest one's tokens are read (the reference's option
    # of this name, default 1 there too): 2 plans and launches step N+1 while step N runs.
    pipeline_depth: int = 1
    # Whole pages of finished and running requests stay matchable by their tokens; a request whose
    # tokens start the same way begins behind them (kairyu/engine/core/radix_kv.py:1-11).
    enable_prefix_caching: bool = False
    # Waiting requests are admitted by (priority, arrival), the lower priority value first, instead
    # of first come, first served (kairyu/engine/core/scheduler.py:191-199, without its aging).
    priority_scheduling: bool = False
    seed: int = 0

    def __post_init__(self) -> None:
        object.__setattr__(self, "dtype", normalize_dtype(self.dtype))
        if self.page_size < 1:
            raise ValueError(f"page_size must be >= 1, got {self.page_size}")
        if self.num_pages is not None and self.num_pages < 2:
            raise ValueError(f"num_pages must be >= 2, got {self.num_pages}")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be >= 1")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_num_partial_prefills < 1:
            raise ValueError("max_num_partial_prefills must be >= 1")
        if self.prefill_chunk_size is not None and self.prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be >= 1")
        if self.decode_mode not in (None, "eager", "cuda_graph"):
            raise ValueError("decode_mode must be None, 'eager' or 'cuda_graph'")
        if self.pipeline_depth not in (1, 2):
            raise ValueError("pipeline_depth must be 1 or 2")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")

    @classmethod
    def from_kwargs(cls, **kwargs: Any) -> "EngineConfig":
        """Exact-key validation: an unknown option is an error, not ignored
        (kairyu/engine/config_validation.py:58-120)."""
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(kwargs) - known)
        if unknown:
            raise TypeError(
                f"unknown engine option(s) {unknown}; known: {sorted(known)}"
            )
        return cls(**kwargs)
