"""Arrangements of norms, mixer and feed-forward around the residual stream."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    Block,
    CacheView,
    LayerSpec,
    Norm,
    StepContext,
    TensorSpec,
)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += ffn(norm(x))`` (kairyu/models/llama.py:88-101).

    The residual is fp32.  Each sub-layer's output is handed on as a pending
    delta and added by the next norm's kernel.

    For a few bf16 rows (decode) the norms have no kernel of their own: the product before a
    norm adds its result to the residual and leaves the rows weighted and their sums of squares
    (``kernels.ResidualNorm``), the product after it scales by the root mean square
    (``kernels.PreNormed``).  That needs norms that offer ``fold_target`` (RMSNorm does) and a
    mixer and feed-forward that offer ``fusable_norm``; any other part gets the plain flow.
    """

    graph_safe = True

    takes_next_norm = True  # forward accepts the norm of the block that runs next

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

    def _fused(self, ctx: StepContext) -> bool:
        if ctx.dtype != torch.bfloat16 or not kernels.fused_norm_available():
            return False
        if not (hasattr(self.mixer_norm, "fold_target") and hasattr(self.ffn_norm, "fold_target")):
            return False  # a norm offers ``fold_target`` when the products around it can take its two halves
        mixer_ok = getattr(self.mixer, "fusable_norm", None)
        ffn_ok = getattr(self.ffn, "fusable_norm", None)
        return bool(mixer_ok and ffn_ok and mixer_ok(ctx.num_tokens) and ffn_ok(ctx.num_tokens))

    def prenorm_target(self, ctx: StepContext) -> Optional[Norm]:
        """The norm the block before this one may fold into its last product, or None."""
        return self.mixer_norm if self._fused(ctx) else None

    def forward(
        self,
        residual: torch.Tensor,
        delta,
        ctx: StepContext,
        cache: CacheView,
        next_norm: Optional[Norm] = None,
    ):
        if isinstance(delta, kernels.PreNormed):  # the block before has added its output and begun our norm
            normed = delta
        else:
            normed = self.mixer_norm.apply(residual, delta, ctx)
        if not self._fused(ctx):
            mixed = self.mixer.forward(normed, ctx, cache)
            normed = self.ffn_norm.apply(residual, mixed, ctx)
            return residual, self.ffn.forward(normed, ctx)
        mixed = self.mixer.forward(normed, ctx, cache, fold=self.ffn_norm.fold_target(residual, ctx, "ffn"))
        fold = next_norm.fold_target(residual, ctx, "mixer") if next_norm is not None else None
        return residual, self.ffn.forward(mixed, ctx, fold=fold)
