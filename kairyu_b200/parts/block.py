"""Arrangements of norms, mixer and feed-forward around the residual stream."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200.parts.base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    Block,
    CacheView,
    LayerSpec,
    StepContext,
    TensorSpec,
)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += ffn(norm(x))`` (kairyu/models/llama.py:88-101).

    The residual is fp32.  Each sub-layer's output is handed on as a pending
    delta and added by the next norm's kernel.
    """

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: str, shared: dict, **_: object) -> None:
        context = dict(dtype=dtype, device=device, shared=shared)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **context)
        self.mixer = MIXERS.build(layer.mixer, **context)
        self.ffn_norm = NORMS.build(layer.ffn_norm, **context)
        self.ffn = FEED_FORWARDS.build(layer.ffn, **context)
        self._parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for part in self._parts for spec in part.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self._parts:
            part.load(tensors)

    def bytes_streamed(self) -> int:
        return sum(part.bytes_streamed() for part in self._parts)

    def forward(
        self,
        residual: torch.Tensor,
        delta: Optional[torch.Tensor],
        ctx: StepContext,
        cache: CacheView,
    ) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
        normed = self.mixer_norm.apply(residual, delta, ctx)
        mixed = self.mixer.forward(normed, ctx, cache)
        normed = self.ffn_norm.apply(residual, mixed, ctx)
        return residual, self.ffn.forward(normed, ctx)
