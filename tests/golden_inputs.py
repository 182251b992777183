"""Seeded weights and prompts shared by the golden script and the tests."""

from __future__ import annotations

from typing import Mapping

import torch

from kairyu_b200.weights.random_init import _specs_without_building, random_tensors
from kairyu_b200.registry import architecture_of


def golden_weights(config: Mapping, seed: int) -> dict[str, torch.Tensor]:
    """fp32 CPU tensors by HF name for a tiny config (the tied head is absent)."""
    architecture = architecture_of(config)
    spec = architecture.build_spec(architecture.parse_config(config))
    return random_tensors(_specs_without_building(spec), seed, device="cpu")


def golden_prompt(config: Mapping, seed: int, length: int = 90) -> list[int]:
    generator = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, config["vocab_size"], (length,), generator=generator).tolist()


def as_held_in_bf16(weights: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The values a bfloat16 engine computes with, as fp32 tensors: matrices and
    biases rounded to bf16, norm weights (stored in 32-bit) left as they are."""
    held = {}
    for name, tensor in weights.items():
        keep = tensor.ndim == 1 and name.endswith("norm.weight")
        held[name] = tensor if keep else tensor.to(torch.bfloat16).float()
    return held


def golden_weights_on(config: Mapping, seed: int, device: str) -> dict[str, torch.Tensor]:
    """As ``golden_weights`` but drawn on ``device`` (a device has its own random stream: these
    are the values ``init_random`` gives a model built there with the same seed)."""
    architecture = architecture_of(config)
    spec = architecture.build_spec(architecture.parse_config(config))
    return random_tensors(_specs_without_building(spec), seed, device=device)
