"""Rotary position encoding: the cos/sin table, computed once in fp32.

Formulas follow kairyu/models/layers.py:93-146 (inverse frequencies from
``arange(0, dim, 2)/dim`` in fp32, llama3 frequency scaling, yarn ramp; the
table holds cos and sin of ``position * inv_freq``).  The reference stores the
half-width table twice side by side (``cat(freqs, freqs)``); here only the
distinct half is kept and the kernel indexes it for both halves of a head.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from kairyu_b200.config.model_config import RopeScaling
from kairyu_b200.parts.base import POSITION_ENCODINGS, PositionEncoding


def _llama3_inv_freq(inv_freq: torch.Tensor, scaling: RopeScaling) -> torch.Tensor:
    """kairyu/models/layers.py:93-104."""
    original = scaling.original_max_position_embeddings
    low_freq_wavelen = original / scaling.low_freq_factor
    high_freq_wavelen = original / scaling.high_freq_factor
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_freq_wavelen, inv_freq / scaling.factor, inv_freq)
    smooth = (original / wavelen - scaling.low_freq_factor) / (
        scaling.high_freq_factor - scaling.low_freq_factor
    )
    smoothed = (1 - smooth) * scaled / scaling.factor + smooth * scaled
    medium = (wavelen >= high_freq_wavelen) & (wavelen <= low_freq_wavelen)
    return torch.where(medium, smoothed, scaled)


def _yarn_mscale(scale: float, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1.0 else 0.1 * mscale * math.log(scale) + 1.0


def _yarn_inv_freq(dim: int, theta: float, scaling: RopeScaling) -> tuple[torch.Tensor, float]:
    """kairyu/models/layers.py:55-81."""
    pos_freqs = theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim)
    extrapolation = 1.0 / pos_freqs
    interpolation = 1.0 / (scaling.factor * pos_freqs)
    original = scaling.original_max_position_embeddings

    def correction_dim(rotations: float) -> float:
        return (dim * math.log(original / (rotations * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(correction_dim(scaling.beta_fast)), 0)
    high = min(math.ceil(correction_dim(scaling.beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2).float() - low) / (high - low)).clamp(0, 1)
    keep = 1.0 - ramp
    inv_freq = interpolation * (1.0 - keep) + extrapolation * keep
    if scaling.mscale is not None and scaling.mscale_all_dim is not None:
        factor = _yarn_mscale(scaling.factor, scaling.mscale) / _yarn_mscale(
            scaling.factor, scaling.mscale_all_dim
        )
    else:
        factor = _yarn_mscale(scaling.factor)
    return inv_freq, factor


def rotary_tables(
    dim: int, theta: float, scaling: Optional[RopeScaling], max_positions: int
) -> tuple[torch.Tensor, torch.Tensor]:
    """(cos, sin), each [max_positions, dim/2] fp32, on the CPU."""
    factor = 1.0
    if scaling is not None and scaling.kind == "yarn":
        inv_freq, factor = _yarn_inv_freq(dim, theta, scaling)
    else:
        inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).to(torch.float32) / dim))
        if scaling is not None and scaling.kind == "llama3":
            inv_freq = _llama3_inv_freq(inv_freq, scaling)
    positions = torch.arange(max_positions, dtype=torch.float32)
    freqs = positions[:, None] * inv_freq[None, :]
    return (freqs.cos() * factor).contiguous(), (freqs.sin() * factor).contiguous()


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(
        self,
        *,
        rotary_dim: int,
        theta: float,
        scaling: Optional[RopeScaling],
        max_positions: int,
        device: str,
        **_: object,
    ) -> None:
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even, got {rotary_dim}")
        self.rotary_dim = rotary_dim
        self.max_positions = max_positions
        cos, sin = rotary_tables(rotary_dim, theta, scaling, max_positions)
        self.cos = cos.to(device)
        self.sin = sin.to(device)

    def rotary_tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin
