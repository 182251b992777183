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


def _yarn_amplitude(factor: float, mscale: float = 1.0) -> float:
    """The factor yarn puts on cos and sin (it stands for a softmax temperature): 1 + 0.1 m ln(s)
    for a context stretched s > 1 times."""
    return 1.0 + 0.1 * mscale * math.log(factor) if factor > 1.0 else 1.0


def _yarn_inv_freq(dim: int, theta: float, scaling: RopeScaling) -> tuple[torch.Tensor, float]:
    """Yarn ("NTK by parts"): pairs of the head that turn often within the original context keep
    their frequency, pairs that turn less than ``beta_slow`` times are slowed ``factor`` times
    (positions interpolated), and the pairs between blend the two linearly in the pair index.
    Pair i has frequency theta^(-2i/dim) and so makes L * theta^(-2i/dim) / 2 pi turns over the
    original context L; solved for i, ``turns`` turns are made by pair
    dim * ln(L / (2 pi turns)) / (2 ln theta).  The blend's ends are that index for ``beta_fast``
    rounded down and for ``beta_slow`` rounded up, as kairyu/models/layers.py:55-81 has them."""
    base = theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim)
    kept, slowed = 1.0 / base, 1.0 / (scaling.factor * base)
    context = scaling.original_max_position_embeddings

    def pair_with(turns: float) -> float:
        return dim * math.log(context / (2 * math.pi * turns)) / (2 * math.log(theta))

    first = max(math.floor(pair_with(scaling.beta_fast)), 0)
    last = min(math.ceil(pair_with(scaling.beta_slow)), dim - 1)
    span = last - first if last != first else 0.001
    slowed_share = ((torch.arange(dim // 2).float() - first) / span).clamp(0, 1)
    inv_freq = slowed * slowed_share + kept * (1.0 - slowed_share)
    amplitude = _yarn_amplitude(scaling.factor)
    if scaling.mscale is not None and scaling.mscale_all_dim is not None:
        amplitude = _yarn_amplitude(scaling.factor, scaling.mscale) / _yarn_amplitude(scaling.factor, scaling.mscale_all_dim)
    return inv_freq, amplitude


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
    graph_safe = True

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
