"""RMSNorm with the residual sum fused in (kairyu/models/layers.py:21-46)."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import NORMS, Norm, StepContext, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """``y = x * rsqrt(mean(x^2) + eps) * weight`` with fp32 statistics."""

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
        tag: str = "norm.out",
    ) -> torch.Tensor:
        count = rows.numel() if rows is not None else residual.shape[0]
        out = ctx.workspace.buffer(tag, count, self.size, self.dtype)
        kernels.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows)
        return out
