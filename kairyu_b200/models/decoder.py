"""The model container: parts built from a :class:`ModelSpec`, run in the order
the spec's schedule gives.  It owns no architecture knowledge."""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200.parts.base import (
    BLOCKS,
    EMBEDDINGS,
    HEADS,
    NORMS,
    POSITION_ENCODINGS,
    CacheView,
    ModelSpec,
    PartSpec,
    StepContext,
    TensorSpec,
)

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def torch_dtype(name: str) -> torch.dtype:
    return _TORCH_DTYPES[name]


class DecoderModel:
    def __init__(self, spec: ModelSpec, *, dtype: str, device: str) -> None:
        self.spec = spec
        self.dtype_name = dtype
        self.dtype = torch_dtype(dtype)
        self.device = device
        shared: dict[Any, Any] = {}
        context = dict(dtype=self.dtype, device=device, shared=shared)
        self.embedding = EMBEDDINGS.build(spec.embedding, **context)
        self.embedding_position = (
            POSITION_ENCODINGS.build(spec.embedding_position, **context) if spec.embedding_position is not None else None
        )
        self.blocks = [
            BLOCKS.build(PartSpec(layer.block), layer=layer, **context) for layer in spec.layers
        ]
        self.final_norm = NORMS.build(spec.final_norm, **context)
        self.head = HEADS.build(spec.head, **context)
        self.schedule = spec.schedule
        self._validate_schedule()

    def _validate_schedule(self) -> None:
        written: set[int] = set()
        for call in self.schedule:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {call.layer}, the model has {len(self.blocks)}")
            if call.writes_cache:
                if call.cache_slot in written:
                    raise ValueError(f"cache slot {call.cache_slot} is written by two calls")
                written.add(call.cache_slot)
            elif call.cache_slot not in written:
                raise ValueError(
                    f"a call reads cache slot {call.cache_slot} before any call has written it"
                )

    # -- weights
    def graph_safe(self) -> bool:
        """Whether a step of prompt portions can be captured in a CUDA graph: every part says so of itself,
        and a block also of the parts it built."""
        def safe(part: Any) -> bool:
            if not getattr(part, "graph_safe", False):
                return False
            return all(safe(inner) for inner in getattr(part, "_parts", ()))

        return all(safe(part) for part in self.parts())

    def parts(self) -> list[Any]:
        extra = [self.embedding_position] if self.embedding_position is not None else []
        return [self.embedding, *extra, *self.blocks, self.final_norm, self.head]

    def tensor_specs(self) -> list[TensorSpec]:
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def bytes_streamed_per_step(self) -> int:
        """Weight bytes a decode step reads: every call's block, the final norm
        and the head (embedding rows are gathered, not streamed)."""
        total = sum(self.blocks[call.layer].bytes_streamed() for call in self.schedule)
        return total + self.final_norm.bytes_streamed() + self.head.bytes_streamed()

    # -- cache needs: slot -> specs of the mixer that writes it
    def cache_slot_specs(self) -> dict[int, tuple[Any, ...]]:
        slots: dict[int, tuple[Any, ...]] = {}
        for call in self.schedule:
            if call.writes_cache:
                slots[call.cache_slot] = tuple(self.blocks[call.layer].mixer.cache_specs())
        return slots

    # -- compute
    def forward(
        self,
        ctx: StepContext,
        cache_views: Mapping[tuple[int, bool], CacheView],
        want_rows: Optional[torch.Tensor],
    ) -> Optional[torch.Tensor]:
        """Run the step's tokens through every scheduled call; return fp32
        logits at ``want_rows`` (flat token indices), or None when none are wanted."""
        residual = self.embedding.forward(ctx)
        if self.embedding_position is not None:
            self.embedding_position.embed_hook(residual, ctx)
        delta: Optional[torch.Tensor] = None
        calls = self.schedule
        for index, call in enumerate(calls):
            view = cache_views[(call.cache_slot, call.writes_cache)]
            block = self.blocks[call.layer]
            if getattr(block, "takes_next_norm", False):
                # a block may begin the first norm of the block that runs next, if that block offers one
                following = self.blocks[calls[index + 1].layer] if index + 1 < len(calls) else None
                offer = getattr(following, "prenorm_target", None)
                residual, delta = block.forward(residual, delta, ctx, view, next_norm=offer(ctx) if offer else None)
            else:
                residual, delta = block.forward(residual, delta, ctx, view)
        if want_rows is None or want_rows.numel() == 0:
            return None
        hidden = self.final_norm.apply(residual, delta, ctx, rows=want_rows)
        return self.head.forward(hidden, ctx)
