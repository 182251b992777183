"""Binds checkpoint tensors to a model's parts by name, with one error that
says everything that is wrong with the file (kairyu/models/loader.py:106-265
raises on the first missing tensor and ignores the rest).

Tensors the model does not ask for are passed over, as the reference does
(``strict=False``, kairyu/models/loader.py:250): exports carry stray buffers.
They are still named in the error when something else is wrong, and
``strict_unexpected=True`` (the ``validate`` command) makes them an error of
their own."""

from __future__ import annotations

import fnmatch
import json
from pathlib import Path
from typing import Any, Sequence

import torch

from kairyu_b200.parts.base import TensorSpec
from kairyu_b200.weights.reader import CheckpointReader

# Buffers some exporters save although they are recomputed at load.
IGNORED_TENSORS = ("*.rotary_emb.inv_freq",)

_FLOAT_TAGS = {"F64", "F32", "F16", "BF16"}
_INT_TAGS = {"I64", "I32", "I16", "I8", "U8"}


class WeightError(ValueError):
    """The checkpoint does not fit the model; lists every mismatch."""

    def __init__(
        self,
        where: str,
        missing: Sequence[str],
        unexpected: Sequence[str],
        wrong_shape: Sequence[tuple[str, tuple[int, ...], tuple[int, ...]]],
        wrong_dtype: Sequence[tuple[str, str, str]],
    ) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"checkpoint {where} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(
                f"  wrong shapes ({len(self.wrong_shape)}): "
                + ", ".join(f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape)
            )
        if self.wrong_dtype:
            lines.append(
                f"  wrong dtypes ({len(self.wrong_dtype)}): "
                + ", ".join(f"{n} is {got}, expected {want}" for n, got, want in self.wrong_dtype)
            )
        super().__init__("\n".join(lines))


def read_config(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise ValueError(f"{model_dir} has no config.json")  # kairyu/models/loader.py:121-122
    config = json.loads(path.read_text())
    if not isinstance(config, dict):
        raise ValueError(f"{path} is not a JSON object")
    return config


def held_dtype(spec: TensorSpec, stored_tag: str, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in: matrices and biases in the compute dtype,
    integer tables as int32, and a ``vector`` stored in 32-bit stays 32-bit."""
    if spec.role == "int_table":
        return torch.int32
    if spec.role == "vector" and stored_tag in ("F32", "F64"):
        return torch.float32
    return compute


def load_into(model: Any, model_dir: str | Path, *, strict_unexpected: bool = False) -> None:
    """Fill every part of ``model`` (a DecoderModel) from ``model_dir``."""
    reader = CheckpointReader(model_dir)
    specs: list[TensorSpec] = model.tensor_specs()
    missing: list[str] = []
    wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = []
    wrong_dtype: list[tuple[str, str, str]] = []
    source_of: dict[str, str] = {}
    for spec in specs:
        source = spec.name
        if source not in reader:
            if spec.alias_of is not None and spec.alias_of in reader:
                source = spec.alias_of
            else:
                missing.append(spec.name)
                continue
        elif spec.alias_of is not None:
            # A tied head: the file's own copy, if any, is not used
            # (kairyu/models/loader.py:228-229, 261-263).
            source = spec.alias_of if spec.alias_of in reader else source
        if reader.shape(source) != tuple(spec.shape):
            wrong_shape.append((source, reader.shape(source), tuple(spec.shape)))
            continue
        tag = reader.stored_dtype(source)
        wanted = _INT_TAGS if spec.role == "int_table" else _FLOAT_TAGS
        if tag not in wanted:
            wrong_dtype.append((source, tag, "an integer type" if spec.role == "int_table" else "a floating type"))
            continue
        source_of[spec.name] = source
    used = set(source_of.values()) | {spec.name for spec in specs}
    unexpected = [
        name
        for name in reader.names()
        if name not in used and not any(fnmatch.fnmatch(name, pattern) for pattern in IGNORED_TENSORS)
    ]
    if missing or wrong_shape or wrong_dtype or (unexpected and strict_unexpected):
        raise WeightError(str(model_dir), missing, unexpected, wrong_shape, wrong_dtype)

    tensors: dict[str, torch.Tensor] = {}
    by_source: dict[tuple[str, torch.dtype], torch.Tensor] = {}
    for spec in specs:
        source = source_of[spec.name]
        dtype = held_dtype(spec, reader.stored_dtype(source), model.dtype)
        key = (source, dtype)
        if key not in by_source:  # a tied head shares the embedding's storage
            by_source[key] = reader.tensor(source).to(device=model.device, dtype=dtype)
        tensors[spec.name] = by_source[key]
    model.load(tensors)
