"""Python entry points of the hand-written sm_100a kernels.

Every function takes CUDA tensors, checks what the kernel assumes, and launches
on the current stream.  There is no other implementation behind them: a tensor
that is not on a CUDA device, or a library that cannot be built or loaded, is
an error.  Model parts call these as ``kernels.<name>(...)``.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from kairyu_b200.kernels.build import KernelBuildError, load_library

# The library products (cuBLAS through torch) may otherwise add split-K partial sums in
# bfloat16; this engine's products accumulate and reduce in fp32.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

c_int = ctypes.c_int
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p

FLAG_BAD_PAGE = 1
FLAG_BAD_TOKEN = 2
FLAG_BAD_ROW = 4
FLAG_BAD_POS = 8
FLAG_TIMEOUT = 16
FLAG_MISALIGNED = 32

_CODES = {
    -1: "bad argument",
    -2: "a size this kernel does not support",
    -3: "a required pointer is null",
}


class KernelError(RuntimeError):
    pass


launch_count = 0  # kernel launches made through this module (library products not counted)


def _check(code: int, what: str, launches: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += launches
        return
    if code < 0:
        raise KernelError(f"{what}: {_CODES.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current stream of the current device.  The raw accessor costs a fraction of a
    microsecond; building a torch Stream object for every launch cost 15 (a step launches hundreds)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _need_cuda(what: str, *tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError(
                f"{what}: tensor on {tensor.device}; the kernels of kairyu_b200 run on CUDA "
                "devices only and have no CPU implementation"
            )


def _is_bf16(tensor: torch.Tensor, what: str) -> int:
    if tensor.dtype == torch.bfloat16:
        return 1
    if tensor.dtype == torch.float32:
        return 0
    raise KernelError(f"{what}: dtype {tensor.dtype} is not supported (float32 or bfloat16)")


def _need_i32(what: str, *tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and (tensor.dtype != torch.int32 or not tensor.is_contiguous()):
            raise KernelError(f"{what}: index tensors must be contiguous int32")


_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(library: str, name: str, argtypes: list) -> ctypes._CFuncPtr:
    function = _functions.get(name)
    if function is None:
        function = getattr(load_library(library), name)
        function.argtypes = argtypes
        function.restype = c_int
        _functions[name] = function
    return function


# ----------------------------------------------------------------------------- elementwise


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, flag: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[ids[t]] as fp32."""
    _need_cuda("embedding", table, ids, out, flag)
    _need_i32("embedding", ids)
    V, H = table.shape
    if out.dtype != torch.float32 or out.shape != (ids.numel(), H) or not out.is_contiguous():
        raise KernelError("embedding: out must be contiguous fp32 [tokens, hidden]")
    if not table.is_contiguous():
        raise KernelError("embedding: table must be contiguous")
    fn = _fn("elementwise", "kb_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(table.data_ptr(), _is_bf16(table, "embedding"), ids.data_ptr(), out.data_ptr(), ids.numel(), H, V, _ptr(flag), _stream()), "embedding")


def patch_tokens(ids: torch.Tensor, source: torch.Tensor, sampled: torch.Tensor, flag: Optional[torch.Tensor] = None) -> None:
    """ids[t] = sampled[source[t]] wherever source[t] >= 0 (tokens the host has not seen yet)."""
    _need_cuda("patch_tokens", ids, source, sampled, flag)
    _need_i32("patch_tokens", ids, source, sampled)
    if source.numel() != ids.numel() or not (ids.is_contiguous() and source.is_contiguous() and sampled.is_contiguous()):
        raise KernelError("patch_tokens: ids and source must be contiguous and of one length")
    fn = _fn("elementwise", "kb_patch_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(fn(ids.data_ptr(), source.data_ptr(), sampled.data_ptr(), ids.numel(), sampled.numel(), _ptr(flag), _stream()), "patch_tokens")


def rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    *,
    delta: Optional[torch.Tensor] = None,
    rows: Optional[torch.Tensor] = None,
) -> None:
    """``x += delta`` (if given and ``rows`` is None), ``out = rmsnorm(x) * weight``.

    With ``rows`` only the listed rows of x (+delta) are normed, into
    out[0..len(rows)), and x is not modified.
    """
    _need_cuda("rmsnorm", x, weight, out, delta, rows)
    _need_i32("rmsnorm", rows)
    H = x.shape[-1]
    R = rows.numel() if rows is not None else x.shape[0]
    if not x.is_contiguous() or not out.is_contiguous() or (delta is not None and not delta.is_contiguous()):
        raise KernelError("rmsnorm: tensors must be contiguous")
    if weight.numel() != H or out.shape[-1] != H or out.shape[0] < R:
        raise KernelError("rmsnorm: shape mismatch")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != x.shape):
        raise KernelError("rmsnorm: delta must have the activation dtype and x's shape")
    fn = _fn("elementwise", "kb_rmsnorm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(
        fn(x.data_ptr(), _is_bf16(x, "rmsnorm"), _ptr(delta), weight.data_ptr(), _is_bf16(weight, "rmsnorm"), out.data_ptr(), _is_bf16(out, "rmsnorm"), _ptr(rows), R, H, float(eps), 1, _stream()),
        "rmsnorm",
    )


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda("swiglu", gate_up, out)
    T, two_i = gate_up.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("swiglu: shape or dtype mismatch")
    if not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("swiglu: tensors must be contiguous")
    fn = _fn("elementwise", "kb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(gate_up.data_ptr(), out.data_ptr(), _is_bf16(out, "swiglu"), T, two_i // 2, _stream()), "swiglu")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda("gather_rows", src, rows, out)
    _need_i32("gather_rows", rows)
    if src.dtype != out.dtype or out.shape != (rows.numel(), src.shape[1]):
        raise KernelError("gather_rows: shape or dtype mismatch")
    if not src.is_contiguous() or not out.is_contiguous():
        raise KernelError("gather_rows: tensors must be contiguous")
    fn = _fn("elementwise", "kb_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(src.data_ptr(), rows.data_ptr(), out.data_ptr(), _is_bf16(src, "gather_rows"), rows.numel(), src.shape[1], _stream()), "gather_rows")


# ----------------------------------------------------------------------------- rope + cache write


def qk_norm_rope_kv_write(
    qkv: torch.Tensor,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    eps: float = 0.0,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
    block_table: Optional[torch.Tensor] = None,
    write_from: Optional[torch.Tensor] = None,
    k_cache: Optional[torch.Tensor] = None,
    v_cache: Optional[torch.Tensor] = None,
    flag: Optional[torch.Tensor] = None,
) -> None:
    """In place on the packed ``qkv`` rows: per-head norm of q and k (if weights
    are given), rotation (if tables are given), then k and v into the paged
    cache (if caches are given)."""
    _need_cuda("qk_norm_rope_kv_write", qkv, positions, row_ids, q_norm_weight, k_norm_weight, cos, sin, block_table, write_from, k_cache, v_cache, flag)
    _need_i32("qk_norm_rope_kv_write", positions, row_ids, block_table, write_from)
    T = qkv.shape[0]
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1:
        raise KernelError(f"qk_norm_rope_kv_write: qkv must be [tokens, {width}] with unit inner stride")
    rot_half = 0
    max_pos = 0
    if cos is not None:
        if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise KernelError("qk_norm_rope_kv_write: cos and sin must be fp32 tables of one shape")
        if not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError("qk_norm_rope_kv_write: cos and sin must be contiguous")
        max_pos, rot_half = cos.shape
    norm_bf16 = 0
    if q_norm_weight is not None:
        if k_norm_weight is None or q_norm_weight.dtype != k_norm_weight.dtype:
            raise KernelError("qk_norm_rope_kv_write: q and k norm weights come together, in one dtype")
        norm_bf16 = _is_bf16(q_norm_weight, "qk_norm_rope_kv_write")
    page_size = num_pages = max_pages = 0
    if k_cache is not None:
        if v_cache is None or k_cache.shape != v_cache.shape or k_cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv_write: caches must match each other and the qkv dtype")
        if not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise KernelError("qk_norm_rope_kv_write: caches must be contiguous")
        num_pages, page_size, kv_heads, dim = k_cache.shape
        if kv_heads != num_kv_heads or dim != head_dim:
            raise KernelError("qk_norm_rope_kv_write: cache geometry does not match the heads")
        if block_table is None or write_from is None:
            raise KernelError("qk_norm_rope_kv_write: a cache write needs block_table and write_from")
        max_pages = block_table.shape[1]
    fn = _fn(
        "rope_kv",
        "kb_qk_norm_rope_kv_write",
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(
            qkv.data_ptr(), _is_bf16(qkv, "qk_norm_rope_kv_write"), T, qkv.stride(0), num_q_heads, num_kv_heads, head_dim,
            _ptr(q_norm_weight), _ptr(k_norm_weight), norm_bf16, float(eps), _ptr(cos), _ptr(sin), rot_half, max_pos,
            positions.data_ptr(), row_ids.data_ptr(), _ptr(block_table), max_pages, _ptr(write_from),
            _ptr(k_cache), _ptr(v_cache), page_size, num_pages, _ptr(flag), _stream(),
        ),
        "qk_norm_rope_kv_write",
    )


# ----------------------------------------------------------------------------- attention


def paged_attention_generic(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    scale: float,
    window: int = 0,
    flag: Optional[torch.Tensor] = None,
) -> None:
    """fp32-arithmetic attention of every token in ``q`` over its request's pages.

    ``q``: [tokens, >= heads*dim] (a view into the packed qkv rows is fine);
    ``out``: [tokens, heads*dim].
    """
    _need_cuda("paged_attention_generic", q, out, k_cache, v_cache, positions, row_ids, block_table, flag)
    _need_i32("paged_attention_generic", positions, row_ids, block_table)
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    if q.dtype != k_cache.dtype or out.dtype != q.dtype or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_generic: dtype or cache shape mismatch")
    if q.stride(1) != 1 or out.stride(1) != 1 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("paged_attention_generic: inner strides must be 1 and caches contiguous")
    if head_dim > 256:
        raise KernelError(f"paged_attention_generic: head_dim {head_dim} > 256 is not supported")
    if num_q_heads % num_kv_heads:
        raise KernelError("paged_attention_generic: query heads must be a multiple of KV heads")
    T = q.shape[0]
    fn = _fn(
        "attention_generic",
        "kb_paged_attention_generic",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            _is_bf16(q, "paged_attention_generic"), positions.data_ptr(), row_ids.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], T, num_q_heads, num_kv_heads, head_dim, page_size, num_pages, float(scale),
            int(window), _ptr(flag), _stream(),
        ),
        "paged_attention_generic",
    )


DECODE_SPLIT = 128  # keys per split of the split-KV kernel (csrc/attention_mma.cu: DEC_SPLIT)


def attention_mma_supported(head_dim: int, num_q_heads: int, num_kv_heads: int) -> bool:
    """Sizes the tensor-core attention kernels take; others use the generic kernel."""
    return (
        head_dim % 16 == 0
        and 16 <= head_dim <= 256
        and num_kv_heads >= 1
        and num_q_heads % num_kv_heads == 0
        and num_q_heads // num_kv_heads <= 16
    )


def attention_prefill_tile_rows(head_dim: int) -> int:
    """Queries per tile the prefill attention kernel expects in its tile list
    (csrc/attention_mma.cuh: prefill_tile_rows)."""
    return 128 if head_dim <= 128 else 64


def attention_prefill_wide_tile_rows(head_dim: int) -> Optional[int]:
    """Queries per tile of the second list the prefill attention takes for long portions (the kernel
    that walks two 128-query tiles a block, csrc/attention_prefill_tc5.cu), or None for head sizes
    it does not cover."""
    return 256 if head_dim == 128 else None


def _check_mma_common(what: str, q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError(f"{what}: bf16 only")
    if k_cache.shape != v_cache.shape or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError(f"{what}: caches must be contiguous and of one shape")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"{what}: inner strides must be 1")
    if q.data_ptr() % 16 or (q.stride(0) * 2) % 16 or k_cache.data_ptr() % 16 or v_cache.data_ptr() % 16:
        raise KernelError(f"{what}: q rows and caches must be 16-byte aligned")


def attention_prefill_mma(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    qo_indptr: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    tile_rows: torch.Tensor,
    tile_starts: torch.Tensor,
    num_tiles: int,
    num_q_heads: int,
    scale: float,
    window: int = 0,
    flag: Optional[torch.Tensor] = None,
    max_seq_len: int = 0,
    workspace: object = None,
    num_splits: Optional[int] = None,
    wide_tiles: Optional[tuple[int, torch.Tensor, torch.Tensor]] = None,
    two_tiles: Optional[bool] = None,
) -> None:
    """Flash attention over query tiles (``attention_prefill_tile_rows`` queries each) of
    rows with several tokens (bf16).

    With ``workspace`` and ``max_seq_len`` (a bound on the rows' lengths) given, the tcgen05 kernel
    may share a tile's keys among several blocks when the tiles alone would leave most of the device
    idle (a short portion of a long prompt); their results meet in fp32 scratch of the workspace and a
    second kernel combines them.  ``num_splits`` overrides the choice (tests).

    ``wide_tiles`` (count, rows, starts of tiles of ``attention_prefill_wide_tile_rows`` queries over the
    same portions): long portions of head size 128 go to the kernel that takes two query tiles a block
    when its grid makes two waves or more; ``two_tiles`` overrides that choice (tests)."""
    what = "attention_prefill_mma"
    _need_cuda(what, q, out, k_cache, v_cache, qo_indptr, seq_lens, block_table, tile_rows, tile_starts)
    _need_i32(what, qo_indptr, seq_lens, block_table, tile_rows, tile_starts)
    _check_mma_common(what, q, out, k_cache, v_cache)
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    if not attention_mma_supported(head_dim, num_q_heads, num_kv_heads):
        raise KernelError(f"{what}: head_dim {head_dim} with {num_q_heads}/{num_kv_heads} heads is not supported")
    if _prefill_tc5_ok(q, out, k_cache, v_cache):  # tcgen05 + TMA: S and O in tensor memory
        fn = _fn(
            "attention_prefill_tc5",
            "kb_attention_prefill_tc5",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
        )
        merged = bool(_fn("attention_prefill_tc5", "kb_attention_prefill_tc5_merged", [c_int, c_int])(head_dim, page_size))
        splits = 1
        if workspace is not None and num_tiles > 0:
            if num_splits is not None:
                splits = int(num_splits)
            elif max_seq_len > 0:
                longest = min(int(max_seq_len), int(window) + 128) if window > 0 else int(max_seq_len)
                splits = _fn("attention_prefill_tc5", "kb_attention_prefill_tc5_splits", [c_int, c_int, c_int, c_int])(head_dim, num_q_heads, int(num_tiles), longest)
        use_two = False
        if wide_tiles is not None and wide_tiles[0] > 0 and head_dim == 128 and splits == 1:
            if two_tiles is None:
                use_two = bool(_fn("attention_prefill_tc5", "kb_attention_prefill_tc5_two_tiles", [c_int] * 5)(
                    head_dim, num_q_heads, int(wide_tiles[0]), page_size, int(max_seq_len)))
            else:
                use_two = bool(two_tiles)
            if use_two:
                _need_cuda(what, wide_tiles[1], wide_tiles[2])
                _need_i32(what, wide_tiles[1], wide_tiles[2])
        part_o = part_ml = None
        if splits > 1:
            slots = splits * int(num_tiles) * 128 * num_q_heads
            part_o = workspace.flat("attn.prefill.part_o", slots * head_dim, torch.float32)
            part_ml = workspace.flat("attn.prefill.part_ml", slots * 2, torch.float32)
        _check(
            fn(
                _tensor_map(q, 128), _cache_map(k_cache), _cache_map(v_cache, bands=merged), out.data_ptr(), out.stride(0),
                qo_indptr.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                tile_rows.data_ptr(), tile_starts.data_ptr(), int(num_tiles), num_q_heads, num_kv_heads, head_dim,
                page_size, num_pages, float(scale), int(window), splits, _ptr(part_o), _ptr(part_ml),
                wide_tiles[1].data_ptr() if use_two else None, wide_tiles[2].data_ptr() if use_two else None,
                int(wide_tiles[0]) if use_two else 0, 1 if use_two else 0, _ptr(flag), _stream(),
            ),
            what,
            launches=2 if splits > 1 else 1,
        )
        return
    fn = _fn(
        "attention_mma",
        "kb_attention_prefill_mma",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            qo_indptr.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1],
            tile_rows.data_ptr(), tile_starts.data_ptr(), int(num_tiles), num_q_heads, num_kv_heads, head_dim,
            page_size, num_pages, float(scale), int(window), _ptr(flag), _stream(),
        ),
        what,
    )


def attention_decode_mma(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    decode_rows: torch.Tensor,
    decode_tokens: torch.Tensor,
    num_rows: int,
    max_seq_len: int,
    num_q_heads: int,
    scale: float,
    window: int = 0,
    workspace: object,
    flag: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
) -> None:
    """Split-KV attention of rows that carry one token (bf16), then the merge.

    ``max_seq_len`` bounds every row's length; it sizes the grid and the scratch
    (``workspace.flat`` gives persistent fp32 buffers).  ``num_splits`` overrides the
    number of splits of the TMA-fed kernel (tests use it to make a block stream many tiles).
    """
    what = "attention_decode_mma"
    _need_cuda(what, q, out, k_cache, v_cache, seq_lens, block_table, decode_rows, decode_tokens)
    _need_i32(what, seq_lens, block_table, decode_rows, decode_tokens)
    _check_mma_common(what, q, out, k_cache, v_cache)
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    if not attention_mma_supported(head_dim, num_q_heads, num_kv_heads):
        raise KernelError(f"{what}: head_dim {head_dim} with {num_q_heads}/{num_kv_heads} heads is not supported")
    if _decode_tma_ok(k_cache, v_cache):  # tiled TMA copies of whole runs of key rows, streamed through a ring
        splits_fn = _fn("attention_decode_tma", "kb_attention_decode_tma_splits", [c_int, c_int, c_int, c_int])
        if num_splits is None:
            num_splits = splits_fn(int(num_rows), num_kv_heads, head_dim, max(1, int(max_seq_len)))
        if num_splits < 1:
            raise KernelError(f"{what}: choosing the number of splits failed with code {num_splits}")
        part_o = workspace.flat("attn.part_o", num_rows * num_q_heads * num_splits * head_dim, torch.float32)
        part_ml = workspace.flat("attn.part_ml", num_rows * num_q_heads * num_splits * 2, torch.float32)
        fn = _fn(
            "attention_decode_tma",
            "kb_attention_decode_tma",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
        )
        joined = _joined_cache_map(k_cache, v_cache)  # keys and values in one copy where the cache allows
        map_k = joined or _cache_map(k_cache, bands=True)
        map_v = joined or _cache_map(v_cache, bands=True)
        _check(
            fn(
                map_k, map_v, q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0),
                seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1], decode_rows.data_ptr(),
                decode_tokens.data_ptr(), int(num_rows), num_q_heads, num_kv_heads, head_dim, page_size, num_pages,
                float(scale), int(window), num_splits, part_o.data_ptr(), part_ml.data_ptr(), 1 if joined else 0, _ptr(flag), _stream(),
            ),
            what,
            launches=_fn("attention_decode_tma", "kb_attention_decode_tma_launches", [c_int])(num_splits),
        )
        return
    num_splits = max(1, -(-int(max_seq_len) // DECODE_SPLIT))
    part_o = workspace.flat("attn.part_o", num_rows * num_q_heads * num_splits * head_dim, torch.float32)
    part_ml = workspace.flat("attn.part_ml", num_rows * num_q_heads * num_splits * 2, torch.float32)
    fn = _fn(
        "attention_mma",
        "kb_attention_decode_mma",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1], decode_rows.data_ptr(),
            decode_tokens.data_ptr(), int(num_rows), num_q_heads, num_kv_heads, head_dim, page_size, num_pages,
            float(scale), int(window), num_splits, part_o.data_ptr(), part_ml.data_ptr(), _ptr(flag), _stream(),
        ),
        what,
        launches=2,
    )


def _prefill_tc5_ok(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> bool:
    head_dim = k_cache.shape[3]
    return (
        head_dim in (64, 128)
        and _decode_tma_ok(k_cache, v_cache)
        and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
        and out.stride(1) == 1 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
    )


def _decode_tma_ok(k_cache: torch.Tensor, v_cache: torch.Tensor) -> bool:
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    return (
        head_dim in (64, 128, 192, 256)
        and page_size >= 8 and page_size & (page_size - 1) == 0
        and all(t.stride(3) == 1 and all(t.stride(i) % 8 == 0 for i in range(3)) and t.data_ptr() % 16 == 0 for t in (k_cache, v_cache))
    )


def _cache_map(cache: torch.Tensor, bands: bool = False) -> int:
    """Host address of a cached TMA descriptor of one layer's key (or value) pages: boxes of one
    64-column band (the prefill kernel's), or with ``bands`` of every band at once (the decode kernel's)."""
    key = ("cache", cache.data_ptr(), tuple(cache.shape), tuple(cache.stride()), bands)
    held = _held_map(key)
    if held is None:
        held = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(held) + 63) & ~63
        ll = ctypes.c_longlong
        fn = _fn("attention_decode_tma", "kb_attention_encode_cache_map", [c_void_p, c_void_p, ll, c_int, c_int, c_int, ll, ll, ll, c_int])
        num_pages, page_size, num_kv_heads, head_dim = cache.shape
        code = fn(address, cache.data_ptr(), num_pages, page_size, num_kv_heads, head_dim, cache.stride(0), cache.stride(1), cache.stride(2), 1 if bands else 0)
        if code != 0:
            raise KernelError(f"tensor map encoding of the cache failed with code {code}")
        _keep_map(key, held)
    return (ctypes.addressof(held) + 63) & ~63


def _joined_cache_map(k_cache: torch.Tensor, v_cache: torch.Tensor) -> int:
    """Host address of a cached TMA descriptor over the keys AND the values of one layer's pages, or 0
    where there is none: head size 64, and values that lie a fixed distance behind the keys with the same
    shape and strides (the cache storage allocates them so).  One copy then brings a run of key rows and
    the value rows of the same positions: at 128 bytes a row the decode kernel is bound by how many
    copies an SM can issue, not by their bytes."""
    if k_cache.shape[3] != 64 or k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        return 0
    gap_bytes = v_cache.data_ptr() - k_cache.data_ptr()
    if gap_bytes <= 0 or gap_bytes % 16 != 0 or gap_bytes >= 1 << 40:
        return 0
    key = ("joined", k_cache.data_ptr(), gap_bytes, tuple(k_cache.shape), tuple(k_cache.stride()))
    held = _held_map(key)
    if held is None:
        held = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(held) + 63) & ~63
        ll = ctypes.c_longlong
        fn = _fn("attention_decode_tma", "kb_attention_encode_joined_map", [c_void_p, c_void_p, ll, ll, c_int, c_int, c_int, ll, ll, ll])
        num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
        code = fn(address, k_cache.data_ptr(), gap_bytes // 2, num_pages, page_size, num_kv_heads, head_dim,
                  k_cache.stride(0), k_cache.stride(1), k_cache.stride(2))
        if code != 0:
            raise KernelError(f"tensor map encoding of the cache's keys and values failed with code {code}")
        _keep_map(key, held)
    return (ctypes.addressof(held) + 63) & ~63


# ----------------------------------------------------------------------------- matrix products


def linear(x, weight: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor], *,
           fold: Optional["ResidualNorm"] = None) -> None:
    """out = x @ weight.T (+ bias).

    float32: this package's own FMA kernel (true 32-bit, fixed summation order).
    bfloat16: the weight-streaming kernel up to 8 rows, else the library product (cuBLAS
    through torch), as the reference's ``F.linear`` is (kairyu/models/packed_linear.py:217);
    accumulation is fp32, ``out`` may be bfloat16 or float32.

    ``x`` may be a :class:`PreNormed` (its rows are scaled in the epilogue) and ``fold`` a
    :class:`ResidualNorm` (the result goes into the residual and towards the next norm instead
    of ``out``); both need the weight-streaming kernel (``fused_norm_shapes_ok``).
    """
    scale_by = x if isinstance(x, PreNormed) else None
    if scale_by is not None or fold is not None:
        values = scale_by.values if scale_by is not None else x
        _need_cuda("linear", values, weight, bias, out)
        if fold is None and (out is None or out.shape != (values.shape[0], weight.shape[0])):
            raise KernelError("linear: out does not fit")
        probe = out if out is not None else fold.values
        if values.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.shape[1] != values.shape[1] or not _skinny_ok(values, weight, bias, probe):
            raise KernelError("linear: a fused norm needs bf16 operands that the weight-streaming kernel takes (at most 16 rows, sizes in steps of 16)")
        if fold is not None and (fold.residual.dtype != torch.float32 or fold.residual.shape != (values.shape[0], weight.shape[0])
                                 or fold.values.shape != fold.residual.shape or fold.values.dtype != torch.bfloat16
                                 or fold.sumsq.numel() < 16 * skinny_blocks(values.shape[0], weight.shape[0])):
            raise KernelError("linear: the residual, values and partial sums of a folded norm do not fit the product")
        _gemm_skinny(values, weight, bias, out, gated=False, scale_by=scale_by, fold=fold)
        return
    _need_cuda("linear", x, weight, bias, out)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    if x.dtype == torch.float32:
        if weight.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("linear: the 32-bit path needs fp32 weights and output")
        if bias is not None and bias.dtype != torch.float32:
            raise KernelError("linear: the 32-bit path needs an fp32 bias")
        if x.stride(1) != 1 or weight.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear: inner strides must be 1")
        fn = _fn("gemm_f32", "kb_gemm_f32", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), M, N, K, _stream()), "linear")
        return
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtypes {x.dtype} / {weight.dtype} are not supported")
    if M == 0:
        return
    if few_rows(M, max(K, N)) and _skinny_ok(x, weight, bias, out):
        _gemm_skinny(x, weight, bias, out, gated=False)
        return
    if out.dtype == torch.bfloat16:
        if bias is not None:
            torch.addmm(bias, x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            out.add_(bias)
    else:
        raise KernelError(f"linear: output dtype {out.dtype} is not supported")


SKINNY_MAX_ROWS = 16  # token rows the weight-streaming product takes (csrc/gemm_skinny.cu)
# ... and up to which the engine uses it.  With two token tiles (9 to 16 rows) the step is 5-7 % faster
# on the library product (plain) and the tcgen05 product (gated) with the norms and the position
# encoding as kernels of their own (measured at 9, 12 and 16 rows; a two-tile variant without
# register spills, one k step a batch, was no faster).
SKINNY_FAST_ROWS = 8
# A narrow model is the exception: at width 2,048 a layer's products are 8 to 67 MB and take 5-15 us each, so
# the three launches a layer that the fusions save weigh more than the second token tile costs (16 layers of
# that width, 12 rows: 1.08 -> 0.96 ms a step; 16 rows: 1.14 -> 1.04).
SKINNY_NARROW_WIDTH = 2048


def few_rows(rows: int, width: Optional[int] = None) -> bool:
    """Whether a step of this many token rows runs on the weight-streaming product and its fusions;
    ``width``: the larger side of the product, or the residual's width for a layer's chain of products."""
    if 1 <= rows <= SKINNY_FAST_ROWS:
        return True
    return width is not None and 1 <= rows <= SKINNY_MAX_ROWS and width <= SKINNY_NARROW_WIDTH


def _skinny_ok(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> bool:
    M, K = x.shape
    return (
        M <= SKINNY_MAX_ROWS
        and K % 16 == 0
        and x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
        and x.stride(0) % 16 == 0 and weight.stride(0) % 16 == 0
        and x.data_ptr() % 32 == 0 and weight.data_ptr() % 32 == 0
        and out.dtype in (torch.bfloat16, torch.float32)
        and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))
    )


def _gemm_skinny(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor], *, gated: bool,
                 scale_by: Optional["PreNormed"] = None, fold: Optional["ResidualNorm"] = None) -> None:
    M, K = x.shape
    N = weight.shape[0]
    if scale_by is None and fold is None:
        fn = _fn("gemm_skinny", "kb_gemm_skinny", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
        _check(
            fn(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), out.data_ptr(),
               1 if out.dtype == torch.float32 else 0, out.stride(0), M, N, K, 1 if gated else 0, _stream()),
            "gemm_skinny",
        )
        return
    fn = _fn(
        "gemm_skinny", "kb_gemm_skinny_fused",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
         c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), _ptr(out),
           1 if out is not None and out.dtype == torch.float32 else 0, out.stride(0) if out is not None else 0, M, N, K, 1 if gated else 0,
           _ptr(scale_by.sumsq) if scale_by is not None else None, scale_by.sumsq.shape[0] if scale_by is not None else 0,
           scale_by.hidden if scale_by is not None else 0, float(scale_by.eps) if scale_by is not None else 0.0,
           fold.residual.data_ptr() if fold is not None else None, fold.residual.stride(0) if fold is not None else 0,
           fold.weight.data_ptr() if fold is not None else None, 1 if fold is not None and fold.weight.dtype == torch.bfloat16 else 0,
           fold.values.data_ptr() if fold is not None else None, fold.values.stride(0) if fold is not None else 0,
           fold.sumsq.data_ptr() if fold is not None else None, _stream()),
        "gemm_skinny",
    )


def linear_weight_streaming(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, gated: bool = False) -> None:
    """The weight-streaming kernel itself, for up to 16 bf16 rows (``linear`` and ``linear_swiglu``
    choose it up to ``SKINNY_FAST_ROWS``); ``gated``: out = silu(x.Wg^T) * (x.Wu^T)."""
    _need_cuda("linear_weight_streaming", x, weight, bias, out)
    n_out = weight.shape[0] // 2 if gated else weight.shape[0]
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.shape[1] != x.shape[1] or out.shape != (x.shape[0], n_out) or not _skinny_ok(x, weight, bias, out):
        raise KernelError("linear_weight_streaming: needs bf16 operands, at most 16 rows, sizes in steps of 16, 32-byte aligned rows")
    _gemm_skinny(x, weight, bias, out, gated=gated)


def linear_rope_ok(x, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, num_q_heads: int,
                   num_kv_heads: int, head_dim: int, cos: Optional[torch.Tensor], k_cache: Optional[torch.Tensor]) -> bool:
    """Whether ``linear_rope`` takes this q | k | v product: bf16, at most 16 rows (the weight-streaming
    kernel), a rotation over the whole head, bf16 caches."""
    values = x.values if isinstance(x, PreNormed) else x
    if cos is None or not values.is_cuda or values.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        return False
    if head_dim % 16 or cos.dtype != torch.float32 or cos.dim() != 2 or cos.shape[1] * 2 != head_dim or not cos.is_contiguous():
        return False
    if weight.shape[0] != (num_q_heads + 2 * num_kv_heads) * head_dim or out.shape != (values.shape[0], weight.shape[0]):
        return False
    if k_cache is not None and (k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous()):
        return False
    return _skinny_ok(values, weight, bias, out)


def linear_rope(x, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, num_q_heads: int, num_kv_heads: int,
                head_dim: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, row_ids: torch.Tensor,
                block_table: Optional[torch.Tensor], write_from: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                v_cache: Optional[torch.Tensor], flag: Optional[torch.Tensor] = None) -> None:
    """The q | k | v product of attention for a few rows with the position encoding and the cache
    write in its epilogue (csrc/gemm_skinny.cu, rope): the q columns of ``out`` get the rotated
    queries; rotated keys and the values go straight to their cache pages (``out``'s k and v
    columns are left as they were).  ``x`` may be a :class:`PreNormed`.  Same arithmetic as
    ``linear`` then ``qk_norm_rope_kv_write`` without per-head norms, except that the product is
    not rounded to bf16 before it is rotated."""
    scale_by = x if isinstance(x, PreNormed) else None
    values = scale_by.values if scale_by is not None else x
    _need_cuda("linear_rope", values, weight, bias, out, cos, sin, positions, row_ids, block_table, write_from, k_cache, v_cache, flag)
    _need_i32("linear_rope", positions, row_ids, *(t for t in (block_table, write_from) if t is not None))
    if not linear_rope_ok(x, weight, bias, out, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, cos=cos, k_cache=k_cache):
        raise KernelError("linear_rope: operands the fused kernel does not take (see linear_rope_ok)")
    if sin.shape != cos.shape or sin.dtype != torch.float32 or not sin.is_contiguous():
        raise KernelError("linear_rope: sin must match cos")
    M, K = values.shape
    if positions.numel() != M or row_ids.numel() != M:
        raise KernelError("linear_rope: one position and one row id per token")
    page_size = num_pages = max_pages = 0
    if k_cache is not None:
        if v_cache is None or block_table is None or write_from is None or v_cache.shape != k_cache.shape or v_cache.dtype != k_cache.dtype or not v_cache.is_contiguous():
            raise KernelError("linear_rope: a cache write needs both caches, the block table and write_from")
        if tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim) or block_table.dim() != 2 or not block_table.is_contiguous():
            raise KernelError("linear_rope: cache or block table layout")
        num_pages, page_size = k_cache.shape[0], k_cache.shape[1]
        max_pages = block_table.shape[1]
    fn = _fn(
        "gemm_skinny", "kb_gemm_skinny_rope",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float,
         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
         c_void_p, c_void_p],
    )
    _check(
        fn(values.data_ptr(), values.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), M, weight.shape[0], K,
           _ptr(scale_by.sumsq) if scale_by is not None else None, scale_by.sumsq.shape[0] if scale_by is not None else 0,
           scale_by.hidden if scale_by is not None else 0, float(scale_by.eps) if scale_by is not None else 0.0,
           cos.data_ptr(), sin.data_ptr(), cos.shape[0], num_q_heads, num_kv_heads, head_dim, positions.data_ptr(), row_ids.data_ptr(),
           _ptr(block_table), max_pages, _ptr(write_from), _ptr(k_cache), _ptr(v_cache), page_size, num_pages, _ptr(flag), _stream()),
        "linear_rope",
    )


# ---- RMSNorm inside the products around it (decode: a norm kernel of its own costs as much as
# a third of the q/k/v product it feeds)


@dataclass
class PreNormed:
    """Rows on their way into an RMSNorm whose work is split between two products: ``values`` =
    bf16(x * norm weight), not yet scaled; ``sumsq[b, m]`` = partial sums of x[m]^2, one per block
    of the product that wrote them.  The product that reads it scales row m by
    rsqrt(sum_b sumsq[b, m] / hidden + eps)."""

    values: torch.Tensor
    sumsq: torch.Tensor
    hidden: int
    eps: float

    @property
    def shape(self) -> torch.Size:
        return self.values.shape


@dataclass
class ResidualNorm:
    """What a product does with its result instead of writing it: add it to the fp32 ``residual`` in
    place, and leave ``values`` and ``sumsq`` of a :class:`PreNormed` for the norm (weight, eps) that follows."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float
    values: torch.Tensor
    sumsq: torch.Tensor

    def result(self) -> PreNormed:
        return PreNormed(self.values, self.sumsq, self.residual.shape[1], self.eps)


def fused_norm_available() -> bool:
    """The products of this module can take the RMSNorm around them into their epilogues."""
    return True


def skinny_blocks(rows: int, out_features: int, gated: bool = False) -> int:
    """Blocks the skinny product is launched with: partial sums per row a ``ResidualNorm`` needs room for."""
    fn = _fn("gemm_skinny", "kb_gemm_skinny_blocks", [c_int, c_int, c_int])
    return int(fn(int(rows), int(out_features), 1 if gated else 0))


def fused_norm_shapes_ok(rows: int, hidden: int, *feature_sizes: int) -> bool:
    """Whether products between ``hidden`` (the width of the residual, which the folding products
    write) and these other sizes can all take the fused path.  The product that scales adds one
    partial sum per block of the product that folded: a residual so wide that the folding product
    is launched with more blocks than it can add up keeps the norm kernel."""
    if not few_rows(rows, hidden) or hidden % 16 != 0 or any(size % 16 != 0 for size in feature_sizes):
        return False
    fits = _fold_fits.get((rows, hidden))
    if fits is None:
        limit = int(_fn("gemm_skinny", "kb_gemm_skinny_max_sum_blocks", [])())
        fits = _fold_fits[(rows, hidden)] = skinny_blocks(rows, hidden) <= limit
    return fits


_fold_fits: dict[tuple[int, int], bool] = {}


TC5_MAX_ROWS = 64  # token rows the tcgen05 weight-streaming product takes (csrc/gemm_tc5.cu)
# Encoded TMA descriptors by what they describe.  A caller takes the host addresses of several of
# them before it launches, so none may be freed while a call is being put together: when the table
# is full it is set aside whole (and only dropped when the next one is full, thousands of
# descriptors later) instead of being cleared.
_TENSOR_MAP_LIMIT = 4096
_tensor_maps: dict[tuple, ctypes.Array] = {}
_tensor_maps_before: dict[tuple, ctypes.Array] = {}


def _keep_map(key: tuple, held: ctypes.Array) -> None:
    global _tensor_maps, _tensor_maps_before
    if len(_tensor_maps) >= _TENSOR_MAP_LIMIT:
        _tensor_maps_before = _tensor_maps
        _tensor_maps = {}
    _tensor_maps[key] = held


def _held_map(key: tuple) -> Optional[ctypes.Array]:
    held = _tensor_maps.get(key)
    if held is None:
        held = _tensor_maps_before.get(key)
        if held is not None:
            _keep_map(key, held)  # in use again: it moves to the current table
    return held


_tc5_scratch: list[torch.Tensor] = []  # old buffers stay alive: captured graphs may still point at them


def _tensor_map(tensor: torch.Tensor, box_rows: int) -> int:
    """Host address of a cached TMA descriptor of a row-major bf16 matrix (boxes of [box_rows, 64])."""
    key = (tensor.data_ptr(), tensor.shape[0], tensor.shape[1], tensor.stride(0), box_rows)
    held = _held_map(key)
    if held is None:
        held = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(held) + 63) & ~63
        fn = _fn("gemm_tc5", "kb_tc5_encode_map", [c_void_p, c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, c_int])
        code = fn(address, tensor.data_ptr(), tensor.shape[0], tensor.shape[1], tensor.stride(0), box_rows)
        if code != 0:
            raise KernelError(f"tensor map encoding failed with code {code}")
        _keep_map(key, held)
    return (ctypes.addressof(held) + 63) & ~63


# The tcgen05 product takes a gated weight from this size on.  Measured at 12 to 64 rows against the library
# product followed by the gate kernel: 201 to 524 MB (hidden 4,096 and 5,120) it is level or up to 5 % ahead,
# at 50 to 100 MB (hidden 2,048 to 3,072: 48 to 72 weight rows a block) it takes 18-32 us where the pair
# takes 12-20: a k step costs it about 600 ns however few rows a block owns, and neither more stages in the
# same shared memory nor another order of the k steps nor other cache hints changed that.
TC5_MIN_WEIGHT_BYTES = 160 << 20


def _tc5_ok(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> bool:
    M, K = x.shape
    return (
        M <= TC5_MAX_ROWS
        and K % 8 == 0
        and x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
        and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
        and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
        and out.dtype in (torch.bfloat16, torch.float32)
        and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))
    )


def _gemm_tc5(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, gated: bool,
              flag: Optional[torch.Tensor] = None) -> None:
    M, K = x.shape
    N = weight.shape[0]
    n_out = N // 2 if gated else N
    splits_fn = _fn("gemm_tc5", "kb_gemm_tc5_splits", [c_int, c_int, c_int])
    splits = splits_fn(n_out, K, 1 if gated else 0)
    partial = None
    if splits > 1:
        need = splits * M * n_out
        if not _tc5_scratch or _tc5_scratch[-1].numel() < need or _tc5_scratch[-1].device != x.device:
            _tc5_scratch.append(torch.empty(max(need, 8 * 1024 * 1024), dtype=torch.float32, device=x.device))
        partial = _tc5_scratch[-1]
    box = 16 if M <= 16 else (32 if M <= 32 else 64)
    rows_fn = _fn("gemm_tc5", "kb_gemm_tc5_rows", [c_int, c_int, c_int])
    rows_per_block = rows_fn(n_out, K, 1 if gated else 0)
    fn = _fn("gemm_tc5", "kb_gemm_tc5", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(
        fn(_tensor_map(weight, rows_per_block), _tensor_map(x, box), out.data_ptr(), 1 if out.dtype == torch.float32 else 0, out.stride(0),
           _ptr(bias), _ptr(partial), M, N, K, 1 if gated else 0, rows_per_block, _ptr(flag), _stream()),
        "gemm_tc5",
        launches=2 if splits > 1 else 1,
    )


def linear_swiglu(x, weight_gate_up: torch.Tensor, out: torch.Tensor, scratch: object) -> None:
    """out = silu(x @ Wg.T) * (x @ Wu.T) with ``weight_gate_up`` = [Wg; Wu] stacked by rows.

    For up to 64 bf16 token rows this is one weight-streaming kernel with the gate in its
    epilogue: the mma.sync skinny kernel up to 8 rows (csrc/gemm_skinny.cu; measured on the
    decode step at 8 rows it is 2 % of the step faster than the tcgen05 kernel, whose fixed
    costs - barrier and tensor-memory set-up, the accumulator read-back - weigh more on a 40 us
    kernel), the tcgen05 + TMA kernel from 9 to 64 rows (csrc/gemm_tc5.cu) where the weight is large
    enough for it (``TC5_MIN_WEIGHT_BYTES``); otherwise a product into ``scratch.buffer(...)`` and the
    gate kernel.
    """
    if isinstance(x, PreNormed):  # its rows are scaled in the epilogue, before the gate
        _need_cuda("linear_swiglu", x.values, weight_gate_up, out)
        if (x.values.dtype != torch.bfloat16 or weight_gate_up.dtype != torch.bfloat16 or out.dtype != torch.bfloat16
                or out.shape != (x.values.shape[0], weight_gate_up.shape[0] // 2) or not _skinny_ok(x.values, weight_gate_up, None, out)):
            raise KernelError("linear_swiglu: a fused norm needs bf16 operands that the weight-streaming kernel takes")
        _gemm_skinny(x.values, weight_gate_up, None, out, gated=True, scale_by=x)
        return
    _need_cuda("linear_swiglu", x, weight_gate_up, out)
    M = x.shape[0]
    two_i = weight_gate_up.shape[0]
    if two_i % 2 or out.shape != (M, two_i // 2):
        raise KernelError("linear_swiglu: shape mismatch")
    if M == 0:
        return
    if x.dtype == torch.bfloat16 and weight_gate_up.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
        if few_rows(M, x.shape[1]) and _skinny_ok(x, weight_gate_up, None, out):
            _gemm_skinny(x, weight_gate_up, None, out, gated=True)
            return
        if _tc5_ok(x, weight_gate_up, None, out) and weight_gate_up.numel() * 2 >= TC5_MIN_WEIGHT_BYTES:
            _gemm_tc5(x, weight_gate_up, None, out, gated=True)
            return
    gate_up = scratch.buffer("ffn.gate_up", M, two_i, x.dtype)
    linear(x, weight_gate_up, None, gate_up)
    swiglu(gate_up, out)


# ----------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda("argmax", logits, out)
    _need_i32("argmax", out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be fp32 with unit inner stride")
    n, V = logits.shape
    fn = _fn("sampling", "kb_argmax", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), n, V, out.data_ptr(), _stream()), "argmax")


def edit_logits(
    logits: torch.Tensor,
    rows: torch.Tensor,
    tokens: torch.Tensor,
    mul: torch.Tensor,
    sub: torch.Tensor,
    mask: torch.Tensor,
) -> None:
    _need_cuda("edit_logits", logits, rows, tokens, mul, sub, mask)
    _need_i32("edit_logits", rows, tokens, mask)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("edit_logits: logits must be fp32 with unit inner stride")
    E = rows.numel()
    if not (tokens.numel() == mul.numel() == sub.numel() == mask.numel() == E):
        raise KernelError("edit_logits: entry arrays must have one length")
    if mul.dtype != torch.float32 or sub.dtype != torch.float32:
        raise KernelError("edit_logits: mul and sub must be fp32")
    fn = _fn("sampling", "kb_edit_logits", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(), tokens.data_ptr(), mul.data_ptr(), sub.data_ptr(), mask.data_ptr(), E, _stream()), "edit_logits")


def logprob_report(
    logits: torch.Tensor,
    rows: torch.Tensor,
    tokens: torch.Tensor,
    k: int,
    values: torch.Tensor,
    indices: torch.Tensor,
    *,
    tokens_by_row: bool,
) -> None:
    """For report r over row ``rows[r]`` of the raw logits: ``values[r, 0]`` = log-softmax of its
    token (``tokens[rows[r]]`` when ``tokens_by_row``, else ``tokens[r]``), ``values[r, 1 + i]`` and
    ``indices[r, i]`` the i-th largest log-softmax value and its token id (ties: the lower id)."""
    _need_cuda("logprob_report", logits, rows, tokens, values, indices)
    _need_i32("logprob_report", rows, tokens, indices)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logprob_report: logits must be fp32 with unit inner stride")
    reports = rows.numel()
    n, V = logits.shape
    k = int(k)
    if k < 0 or values.dtype != torch.float32 or not values.is_contiguous() or values.shape != (reports, k + 1):
        raise KernelError("logprob_report: values must be contiguous fp32 [reports, k + 1]")
    if not indices.is_contiguous() or indices.shape != (reports, k):
        raise KernelError("logprob_report: indices must be contiguous int32 [reports, k]")
    if tokens.numel() < (n if tokens_by_row else reports):
        raise KernelError("logprob_report: too few tokens")
    if reports == 0:
        return
    need_fn = _fn("sampling", "kb_logprob_report_scratch_floats", [c_int, c_int, c_int])
    need_fn.restype = ctypes.c_longlong
    scratch = torch.empty(max(1, int(need_fn(reports, V, k))), dtype=torch.float32, device=logits.device)  # the chunks' candidates
    fn = _fn("sampling", "kb_logprob_report", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(
        fn(logits.data_ptr(), logits.stride(0), n, V, rows.data_ptr(), tokens.data_ptr(), 1 if tokens_by_row else 0, reports, k,
           values.data_ptr(), indices.data_ptr() if k else None, scratch.data_ptr(), _stream()),
        "logprob_report",
        launches=2,
    )


def sample_work_floats(rows: int, vocab: int) -> int:
    """Scratch floats ``sample`` needs: the rows' probabilities and the state of its three stages."""
    fn = _fn("sampling", "kb_sample_extra_floats", [c_int])
    return rows * vocab + 1 + int(fn(int(rows)))


def sample(
    logits: torch.Tensor,
    work: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    min_p: torch.Tensor,
    seeds: torch.Tensor,
    out: torch.Tensor,
) -> None:
    """One draw per row; ``seeds`` are int64 bit patterns of the per-position seeds."""
    _need_cuda("sample", logits, work, temperature, top_k, top_p, min_p, seeds, out)
    _need_i32("sample", top_k, out)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be fp32 with unit inner stride")
    if work.dtype != torch.float32 or not work.is_contiguous() or work.numel() < sample_work_floats(n, V) or work.data_ptr() % 8:
        raise KernelError("sample: work must be contiguous fp32 with at least sample_work_floats(rows, vocab) elements")
    if seeds.dtype != torch.int64 or temperature.dtype != torch.float32 or top_p.dtype != torch.float32 or min_p.dtype != torch.float32:
        raise KernelError("sample: parameter dtypes are fp32 (temperature, top_p, min_p), int32 (top_k), int64 (seeds)")
    fn = _fn("sampling", "kb_sample", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(
        fn(logits.data_ptr(), logits.stride(0), work.data_ptr(), n, V, temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), seeds.data_ptr(), out.data_ptr(), _stream()),
        "sample",
    )


__all__ = [
    "few_rows",
    "linear_weight_streaming",
    "linear_rope",
    "linear_rope_ok",
    "logprob_report",
    "KernelBuildError",
    "KernelError",
    "PreNormed",
    "ResidualNorm",
    "argmax",
    "attention_decode_mma",
    "attention_mma_supported",
    "attention_prefill_tile_rows",
    "attention_prefill_wide_tile_rows",
    "attention_prefill_mma",
    "edit_logits",
    "embedding",
    "fused_norm_available",
    "fused_norm_shapes_ok",
    "gather_rows",
    "linear",
    "linear_swiglu",
    "patch_tokens",
    "paged_attention_generic",
    "qk_norm_rope_kv_write",
    "rmsnorm",
    "sample",
    "sample_work_floats",
    "skinny_blocks",
    "swiglu",
]
