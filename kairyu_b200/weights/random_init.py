"""Random weights from a configuration and a seed: in memory, or written as a
model folder (config.json + model.safetensors) that the loader reads back.

Tensors are drawn in the order the model lists them, each from its own
generator seeded by (seed, position in that order), so a seed fixes every
tensor whatever the others' sizes.  Matrices and biases ~N(0, 0.02); norm
weights 1 + N(0, 0.1).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch
from safetensors.torch import save_file

from kairyu_b200.parts.base import TensorSpec

_SAVE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _draw(spec: TensorSpec, seed: int, index: int, device: str) -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed((int(seed) * 1_000_003 + index) & 0x7FFF_FFFF_FFFF_FFFF)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    values = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device)
    if spec.init == "norm":
        return 1.0 + 0.1 * values
    if spec.init == "normal":
        return 0.02 * values
    raise ValueError(f"unknown init {spec.init!r} for {spec.name}")


def random_tensors(specs: list[TensorSpec], seed: int, *, device: str = "cpu") -> dict[str, torch.Tensor]:
    """fp32 tensors for every spec that is not an alias of another one."""
    tensors: dict[str, torch.Tensor] = {}
    for index, spec in enumerate(specs):
        if spec.alias_of is not None:
            continue
        if spec.role == "int_table":
            raise ValueError(f"{spec.name}: integer tables have no random initialisation")
        tensors[spec.name] = _draw(spec, seed, index, device)
    return tensors


def init_random(model: Any, seed: int) -> None:
    """Fill a built model with random weights on its own device (no files)."""
    from kairyu_b200.weights.loading import held_dtype

    specs: list[TensorSpec] = model.tensor_specs()
    tensors: dict[str, torch.Tensor] = {}
    for index, spec in enumerate(specs):
        if spec.alias_of is not None:
            continue
        dtype = held_dtype(spec, "F32" if model.dtype == torch.float32 else "BF16", model.dtype)
        tensors[spec.name] = _draw(spec, seed, index, model.device).to(dtype)
    for spec in specs:
        if spec.alias_of is not None:
            tensors[spec.name] = tensors[spec.alias_of]
    model.load(tensors)


def write_random_model(
    config: Mapping[str, Any], out_dir: str | Path, *, seed: int, dtype: str = "float32"
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a random model."""
    from kairyu_b200.models.decoder import DecoderModel
    from kairyu_b200.registry import architecture_of

    if dtype not in _SAVE_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_SAVE_DTYPES)}")
    architecture = architecture_of(config)
    spec = architecture.build_spec(architecture.parse_config(config))
    specs = _specs_without_building(spec)
    tensors = {
        name: tensor.to(_SAVE_DTYPES[dtype]).contiguous()
        for name, tensor in random_tensors(specs, seed, device="cpu").items()
    }
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    written = dict(config)
    written["dtype"] = dtype
    written.pop("torch_dtype", None)
    (out / "config.json").write_text(json.dumps(written, indent=2, sort_keys=True) + "\n")
    save_file(tensors, str(out / "model.safetensors"), metadata={"format": "pt"})
    return out


def _specs_without_building(spec: Any) -> list[TensorSpec]:
    """Tensor specs of a model spec.  Parts are built on the ``meta`` device, so
    nothing the size of the model is allocated."""
    from kairyu_b200.models.decoder import DecoderModel

    return DecoderModel(spec, dtype="float32", device="meta").tensor_specs()
