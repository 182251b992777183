"""Reads tensors by name from a model folder: ``model.safetensors``, any other
``*.safetensors`` files, or the shards an index names
(kairyu/engine/core/weights.py:36-259)."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open


class CheckpointReader:
    def __init__(self, model_dir: str | Path) -> None:
        self.model_dir = Path(model_dir)
        if not self.model_dir.is_dir():
            raise FileNotFoundError(f"model folder {self.model_dir} does not exist")
        self._file_of: dict[str, Path] = {}
        index = self.model_dir / "model.safetensors.index.json"
        if index.exists():
            weight_map = json.loads(index.read_text()).get("weight_map")
            if not isinstance(weight_map, dict) or not weight_map:
                raise ValueError(f"{index} has no weight_map")
            root = self.model_dir.resolve()
            for name, shard in weight_map.items():
                path = (self.model_dir / shard).resolve()
                if root not in path.parents:
                    raise ValueError(f"{index} names a shard outside the model folder: {shard!r}")
                if not path.exists():
                    raise FileNotFoundError(f"{index} names a missing shard: {shard!r}")
                self._file_of[name] = path
            files = sorted(set(self._file_of.values()))
        else:
            files = sorted(self.model_dir.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"no *.safetensors file in {self.model_dir}")
        self._meta: dict[str, tuple[tuple[int, ...], str]] = {}
        for path in files:
            with safe_open(str(path), framework="pt", device="cpu") as handle:
                for name in handle.keys():
                    if index.exists() and self._file_of.get(name) != path:
                        continue  # a shard may hold tensors the index gives to another file
                    view = handle.get_slice(name)
                    self._meta[name] = (tuple(view.get_shape()), str(view.get_dtype()))
                    self._file_of.setdefault(name, path)
        if index.exists():
            absent = sorted(set(weight_map) - set(self._meta))
            if absent:
                raise ValueError(f"{index} lists tensors its shards do not hold: {absent[:8]}")

    def names(self) -> list[str]:
        return sorted(self._meta)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._meta[name][0]

    def stored_dtype(self, name: str) -> str:
        """safetensors dtype tag: F32, BF16, F16, I32, I64, ..."""
        return self._meta[name][1]

    def __contains__(self, name: str) -> bool:
        return name in self._meta

    def tensor(self, name: str) -> torch.Tensor:
        with safe_open(str(self._file_of[name]), framework="pt", device="cpu") as handle:
            return handle.get_tensor(name)
