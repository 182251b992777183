"""Token embedding and output head (kairyu/models/llama.py:217, 261-273, 612-614)."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import EMBEDDINGS, HEADS, Part, StepContext, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """``x = E[token_ids]``, no scaling; the residual it starts is fp32."""

    graph_safe = True

    def __init__(self, *, name: str, vocab_size: int, hidden_size: int, dtype: torch.dtype, device: str, **_: object) -> None:
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        out = ctx.workspace.buffer("residual", ctx.num_tokens, self.hidden_size, torch.float32)
        kernels.embedding(self.weight, ctx.token_ids, out, ctx.error_flag)
        return out


@HEADS.register("linear_head")
class LinearHead(Part):
    """``logits = h @ W^T`` in fp32 output; ``tied_to`` names the embedding
    tensor to share when the file has no head tensor of its own."""

    graph_safe = True

    def __init__(
        self,
        *,
        name: str,
        vocab_size: int,
        hidden_size: int,
        tied_to: Optional[str],
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), alias_of=self.tied_to)]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def bytes_streamed(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, hidden: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = ctx.workspace.buffer("logits", hidden.shape[0], self.vocab_size, torch.float32)
        kernels.linear(hidden, self.weight, None, logits)
        return logits
