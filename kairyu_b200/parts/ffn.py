"""SiLU-gated feed-forward (kairyu/models/layers.py:193-244):
``down(silu(gate(x)) * up(x))``.  gate and up are one matrix product over the
row-concatenated weight (the reference runs them as two)."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import FEED_FORWARDS, FeedForward, StepContext, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        intermediate_size: int,
        activation: str,
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        if activation != "silu":
            raise ValueError(f"gated feed-forward activation {activation!r} is not implemented (silu)")
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.dtype = dtype
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        return [
            TensorSpec(f"{p}.gate_proj.weight", (self.intermediate_size, self.hidden_size)),
            TensorSpec(f"{p}.up_proj.weight", (self.intermediate_size, self.hidden_size)),
            TensorSpec(f"{p}.down_proj.weight", (self.hidden_size, self.intermediate_size)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat(
            [tensors[f"{p}.gate_proj.weight"], tensors[f"{p}.up_proj.weight"]], dim=0
        ).contiguous()
        self.w_down = tensors[f"{p}.down_proj.weight"].contiguous()

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def fusable_norm(self, tokens: int) -> bool:
        """Whether both products can take the norms around them into their epilogues."""
        return kernels.fused_norm_shapes_ok(tokens, self.hidden_size, self.intermediate_size)

    def forward(self, x, ctx: StepContext, fold=None):
        """``x``: rows, or a ``kernels.PreNormed``; ``fold`` (a ``kernels.ResidualNorm``): the down
        product adds its result to the residual and returns the ``PreNormed`` for the next norm."""
        tokens = x.shape[0]
        ws = ctx.workspace
        hidden = ws.buffer("ffn.hidden", tokens, self.intermediate_size, self.dtype)
        kernels.linear_swiglu(x, self.w_gate_up, hidden, ws)
        if fold is not None:
            kernels.linear(hidden, self.w_down, None, None, fold=fold)
            return fold.result()
        out = ws.buffer("ffn.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(hidden, self.w_down, None, out)
        return out
