"""RMSNorm with the residual sum fused in (kairyu/models/layers.py:21-46)."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import NORMS, Norm, StepContext, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """``y = x * rsqrt(mean(x^2) + eps) * weight`` with fp32 statistics."""

    graph_safe = True

    def __init__(self, *, name: str, size: int, eps: float, dtype: torch.dtype, device: str, **_: object) -> None:
        self.name = name  # full tensor name of the weight
        self.size = size
        self.eps = float(eps)
        self.dtype = dtype
        self.device = device
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), role="vector", init="norm")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()

    def bytes_streamed(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def apply(
        self,
        residual: torch.Tensor,
        delta: Optional[torch.Tensor],
        ctx: StepContext,
        *,
        rows: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        count = rows.numel() if rows is not None else residual.shape[0]
        # a subset of rows (the model's last norm, at the wanted places) has a buffer of its own
        out = ctx.workspace.buffer("norm.out" if rows is None else "norm.rows.out", count, self.size, self.dtype)
        kernels.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows)
        return out

    def fold_target(self, residual: torch.Tensor, ctx: StepContext, tag: str) -> "kernels.ResidualNorm":
        """For a product that takes this norm's first half into its epilogue: it adds its result
        to ``residual`` and leaves the rows weighted and their sums of squares; the product that
        reads them scales by the root mean square (kernels.ResidualNorm / kernels.PreNormed)."""
        rows = residual.shape[0]
        values = ctx.workspace.buffer(f"norm.fold.{tag}.values", rows, self.size, torch.bfloat16)
        sumsq = ctx.workspace.flat(f"norm.fold.{tag}.sumsq", 16 * kernels.skinny_blocks(rows, self.size), torch.float32).view(-1, 16)
        return kernels.ResidualNorm(residual, self.weight, self.eps, values, sumsq)
