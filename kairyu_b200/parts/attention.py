"""Grouped-query attention over the paged cache (kairyu/models/attention.py:24-271).

One matrix product for q|k|v (the reference packs them the same way,
kairyu/models/packed_linear.py:105-122), one kernel for per-head q/k norm +
rotation + cache write, attention over the block table, one product for o.
Sizes, the optional q/k norm, biases, the scale, the window and the position
encoding are constructor arguments; the part does not know its model.
"""

from __future__ import annotations

import contextlib
import math
from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import (
    MIXERS,
    POSITION_ENCODINGS,
    CacheView,
    Mixer,
    PagedKVSpec,
    PartSpec,
    StepContext,
    TensorSpec,
)


OVERLAP_MIXED_ATTENTION = True


class _SideStream:
    """A second stream for work that may run beside the step's own, and the two events that fence it."""

    def __init__(self, device: torch.device) -> None:
        self.stream = torch.cuda.Stream(device=device)
        self.fork = torch.cuda.Event()
        self.join = torch.cuda.Event()


_side_streams: dict[torch.device, _SideStream] = {}


def _side_stream(device: torch.device) -> _SideStream:
    held = _side_streams.get(device)
    if held is None:
        held = _side_streams[device] = _SideStream(device)
    return held


def run_paged_attention(
    qkv: torch.Tensor,
    out: torch.Tensor,
    cache: CacheView,
    ctx: StepContext,
    *,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int,
) -> None:
    """Attention of every token of the step; picks the kernels for the dtype.

    float32: the fp32 kernel for all tokens (its arithmetic per token does not
    depend on the batch).  bfloat16: tensor-core kernels, query tiles for
    rows with several tokens and split-KV for rows with one token; sizes those
    refuse go to the fp32-arithmetic kernel.
    """
    block_table = ctx.block_tables[cache.group]
    use_mma = (
        qkv.dtype == torch.bfloat16
        and kernels.attention_mma_supported(head_dim, num_q_heads, num_kv_heads)
        and not ctx.extras.get("force_generic_attention", False)
    )
    if not use_mma:
        kernels.paged_attention_generic(
            qkv,
            out,
            cache.k,
            cache.v,
            positions=ctx.positions,
            row_ids=ctx.row_ids,
            block_table=block_table,
            num_q_heads=num_q_heads,
            scale=scale,
            window=window,
            flag=ctx.error_flag,
        )
        return
    num_tiles, tile_rows, tile_starts = ctx.tiles[kernels.attention_prefill_tile_rows(head_dim)]
    # A step with prompt portions beside decoded tokens: the two kernels read the same q|k|v rows and
    # write different rows of `out`, and neither fills the device alone (a 512-token portion is 256
    # blocks of tensor-core work, sixteen decode rows a memory-bound stream), so the single-token rows
    # go to a second stream between two events.
    beside = None
    if OVERLAP_MIXED_ATTENTION and num_tiles and ctx.num_decode_rows and qkv.is_cuda and not torch.cuda.is_current_stream_capturing():
        beside = _side_stream(qkv.device)
        beside.fork.record()
        beside.stream.wait_event(beside.fork)
    if num_tiles:
        kernels.attention_prefill_mma(
            qkv,
            out,
            cache.k,
            cache.v,
            qo_indptr=ctx.qo_indptr,
            seq_lens=ctx.seq_lens,
            block_table=block_table,
            tile_rows=tile_rows,
            tile_starts=tile_starts,
            num_tiles=num_tiles,
            num_q_heads=num_q_heads,
            scale=scale,
            window=window,
            flag=ctx.error_flag,
            max_seq_len=ctx.max_portion_seq_len,
            workspace=ctx.workspace,
            wide_tiles=ctx.tiles.get(kernels.attention_prefill_wide_tile_rows(head_dim)),
        )
    if ctx.num_decode_rows:
        with torch.cuda.stream(beside.stream) if beside is not None else contextlib.nullcontext():
            kernels.attention_decode_mma(
                qkv,
                out,
                cache.k,
                cache.v,
                seq_lens=ctx.seq_lens,
                block_table=block_table,
                decode_rows=ctx.decode_rows,
                decode_tokens=ctx.decode_tokens,
                num_rows=ctx.num_decode_rows,
                max_seq_len=ctx.max_seq_len,
                num_q_heads=num_q_heads,
                scale=scale,
                window=window,
                workspace=ctx.workspace,
                flag=ctx.error_flag,
            )
            if beside is not None:
                beside.join.record()
        if beside is not None:
            torch.cuda.current_stream().wait_event(beside.join)


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qk_norm: bool,
        norm_eps: float,
        qkv_bias: bool,
        o_bias: bool,
        position: Optional[PartSpec],
        window: Optional[int] = None,
        scale: Optional[float] = None,
        dtype: torch.dtype,
        device: str,
        shared: dict[Any, Any],
        **_: object,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.qk_norm = qk_norm
        self.norm_eps = float(norm_eps)
        self.qkv_bias = qkv_bias
        self.o_bias = o_bias
        self.window = window
        # kairyu/engine/core/attention/torch_backend.py:64-70 uses SDPA's default 1/sqrt(D)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.dtype = dtype
        self.device = device
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.qkv_width = self.q_size + 2 * self.kv_size
        self.position = None
        if position is not None:
            key = ("position", position)
            if key not in shared:  # one table for all layers that ask for the same encoding
                shared[key] = POSITION_ENCODINGS.build(position, device=device, dtype=dtype)
            self.position = shared[key]
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None

    # -- weights
    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        specs = [
            TensorSpec(f"{p}.q_proj.weight", (self.q_size, self.hidden_size)),
            TensorSpec(f"{p}.k_proj.weight", (self.kv_size, self.hidden_size)),
            TensorSpec(f"{p}.v_proj.weight", (self.kv_size, self.hidden_size)),
            TensorSpec(f"{p}.o_proj.weight", (self.hidden_size, self.q_size)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(f"{p}.q_proj.bias", (self.q_size,), role="bias", init="normal"),
                TensorSpec(f"{p}.k_proj.bias", (self.kv_size,), role="bias", init="normal"),
                TensorSpec(f"{p}.v_proj.bias", (self.kv_size,), role="bias", init="normal"),
            ]
        if self.o_bias:
            specs.append(TensorSpec(f"{p}.o_proj.bias", (self.hidden_size,), role="bias", init="normal"))
        if self.qk_norm:
            specs += [
                TensorSpec(f"{p}.q_norm.weight", (self.head_dim,), role="vector", init="norm"),
                TensorSpec(f"{p}.k_norm.weight", (self.head_dim,), role="vector", init="norm"),
            ]
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_qkv = torch.cat(
            [tensors[f"{p}.q_proj.weight"], tensors[f"{p}.k_proj.weight"], tensors[f"{p}.v_proj.weight"]], dim=0
        ).contiguous()
        self.w_o = tensors[f"{p}.o_proj.weight"].contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat(
                [tensors[f"{p}.q_proj.bias"], tensors[f"{p}.k_proj.bias"], tensors[f"{p}.v_proj.bias"]], dim=0
            ).contiguous()
        if self.o_bias:
            self.b_o = tensors[f"{p}.o_proj.bias"].contiguous()
        if self.qk_norm:
            self.q_norm_weight = tensors[f"{p}.q_norm.weight"].contiguous()
            self.k_norm_weight = tensors[f"{p}.k_norm.weight"].contiguous()
            if self.q_norm_weight.dtype != self.k_norm_weight.dtype:
                self.q_norm_weight = self.q_norm_weight.float()
                self.k_norm_weight = self.k_norm_weight.float()

    def bytes_streamed(self) -> int:
        total = 0
        for tensor in (self.w_qkv, self.b_qkv, self.w_o, self.b_o, self.q_norm_weight, self.k_norm_weight):
            if tensor is not None:
                total += tensor.numel() * tensor.element_size()
        return total

    # -- cache
    def cache_specs(self) -> tuple[Any, ...]:
        return (PagedKVSpec(self.num_kv_heads, self.head_dim, self.window),)

    def query_tile_sizes(self) -> tuple[int, ...]:
        wide = kernels.attention_prefill_wide_tile_rows(self.head_dim)
        return (kernels.attention_prefill_tile_rows(self.head_dim),) + ((wide,) if wide else ())

    # -- compute
    def fusable_norm(self, tokens: int) -> bool:
        """Whether the q/k/v and the output product can take the norms around them into their epilogues."""
        return kernels.fused_norm_shapes_ok(tokens, self.hidden_size, self.q_size)

    def forward(self, x, ctx: StepContext, cache: CacheView, fold=None):
        """``x``: rows, or a ``kernels.PreNormed``; ``fold`` (a ``kernels.ResidualNorm``): the output
        product adds its result to the residual and returns the ``PreNormed`` for the next norm."""
        tokens = x.shape[0]
        ws = ctx.workspace
        qkv = ws.buffer("attn.qkv", tokens, self.qkv_width, self.dtype)
        tables = self.position.rotary_tables() if self.position is not None else None
        cos, sin = tables if tables is not None else (None, None)
        writes = cache.writes
        placement = dict(
            positions=ctx.positions,
            row_ids=ctx.row_ids,
            block_table=ctx.block_tables[cache.group] if writes else None,
            write_from=ctx.write_from if writes else None,
            k_cache=cache.k if writes else None,
            v_cache=cache.v if writes else None,
            flag=ctx.error_flag,
        )
        heads = dict(num_q_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim)
        if not self.qk_norm and kernels.few_rows(tokens, self.hidden_size) and kernels.linear_rope_ok(x, self.w_qkv, self.b_qkv, qkv, cos=cos, k_cache=placement["k_cache"], **heads):
            # a few bf16 rows: the rotation and the cache write ride in the product's epilogue
            kernels.linear_rope(x, self.w_qkv, self.b_qkv, qkv, cos=cos, sin=sin, **heads, **placement)
        else:
            kernels.linear(x, self.w_qkv, self.b_qkv, qkv)
            kernels.qk_norm_rope_kv_write(
                qkv,
                self.num_heads,
                self.num_kv_heads,
                self.head_dim,
                q_norm_weight=self.q_norm_weight,
                k_norm_weight=self.k_norm_weight,
                eps=self.norm_eps,
                cos=cos,
                sin=sin,
                **placement,
            )
        mixed = ws.buffer("attn.mixed", tokens, self.q_size, self.dtype)
        run_paged_attention(
            qkv,
            mixed,
            cache,
            ctx,
            num_q_heads=self.num_heads,
            num_kv_heads=self.num_kv_heads,
            head_dim=self.head_dim,
            scale=self.scale,
            window=self.window or 0,
        )
        if fold is not None:
            kernels.linear(mixed, self.w_o, self.b_o, None, fold=fold)
            return fold.result()
        out = ws.buffer("attn.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(mixed, self.w_o, self.b_o, out)
        return out
