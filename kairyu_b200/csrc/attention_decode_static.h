// kb_attention_decode_mma_static: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in ytworks/kairyu; it exists for callers of
// this library that must not (or cannot) allocate device memory around the call.
//
// Who that is.  The ordinary entry point, kb_attention_decode_mma, is handed two
// scratch buffers for the per-split partial results, and somebody has to allocate
// them.  Some callers have no allocator to ask: a host program that gave all of
// the device's memory to its own pool at start-up and hands out none of it at run
// time; a plug-in loaded into a process whose allocator it has no access to; code
// running where cudaMalloc's implicit device-wide synchronisation is not
// acceptable; a C caller with no torch in the process at all.  They pass only
// inputs and the output here.
//
// How.  The scratch is a file-scope `static __device__` array inside the library,
// KB_STATIC_SCRATCH_FLOATS floats (16 MiB) per GPU that loads the library, held
// until the process exits.  The call needs
//     num_rows * Hq * num_splits * (D + 2)   floats,   num_splits = ceil(max_seq_len / 128),
// and returns KB_ERR_SCRATCH_TOO_SMALL (-4) without launching anything when that
// exceeds the array (8 rows of 32 heads of 128 at 8,192 tokens of context fit;
// 64 such rows fit up to 1,024 tokens).
//
// Set-up.  The first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it; make that
// first call outside any stream capture.  The call itself calls no cudaMalloc,
// cudaFree or allocating library routine.
//
// Sharing.  Every call on a device uses the same array and finds the previous
// call's contents in it.  Nothing has to start at zero: each (row, head, split)
// entry that the merge step reads is written by the split step of the same call
// first.  Two calls that overlap on the GPU (different streams, or a graph
// replayed while another call runs) would write the same scratch: keep calls on
// one stream or otherwise ordered.
#pragma once

#include <cuda_runtime.h>

#define KB_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define KB_ERR_SCRATCH_TOO_SMALL (-4)
#define KB_ERR_SETUP_FAILED (-5)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as kb_attention_decode_mma, without the two scratch pointers and
// with max_seq_len in place of num_splits.
//   q:   [tokens, q_stride] bf16, query of row i at q[decode_tokens[i]]
//   out: [tokens, out_stride] bf16
//   k_cache, v_cache: [num_pages, page_size, Hkv, D] bf16
//   seq_lens: [rows_total] int32; block_table: [rows_total, max_pages] int32
//   decode_rows, decode_tokens: [num_rows] int32
// Requirements, checked before anything is launched (KB_ERR_BAD_ARG, -1, if one fails;
// KB_ERR_NULL, -3, for a null pointer; KB_ERR_UNSUPPORTED_SIZE, -2, for a head size that is
// no multiple of 16 or beyond 256):
//   - q, k_cache and v_cache start on 16-byte boundaries; q_stride is a multiple of 8
//     elements; q_stride and out_stride are at least Hq * D; inner strides are 1;
//   - the caches are contiguous in the layout above (a page of one cache is a contiguous
//     [page_size, Hkv * D] tile);
//   - page_size, max_pages, num_pages >= 1; window >= 0 (0: every key); Hq a multiple of
//     Hkv with at most 16 query heads per KV head.
// Not checked: that block_table entries lie in [0, num_pages).  A page outside the pool is
// skipped (never read); the row's output then misses those keys, and this entry point has no
// error word to report it in.  Keep tables valid.
// Returns 0, a negative KB_ERR_* code, or a positive cudaError_t.
int kb_attention_decode_mma_static(const void* q, int q_stride, void* out, int out_stride,
                                   const void* k_cache, const void* v_cache, const int* seq_lens,
                                   const int* block_table, int max_pages, const int* decode_rows,
                                   const int* decode_tokens, int num_rows, int Hq, int Hkv, int D,
                                   int page_size, int num_pages, float scale, int window,
                                   int max_seq_len, cudaStream_t stream);

// Floats of scratch the library holds per device (KB_STATIC_SCRATCH_FLOATS).
int kb_attention_decode_static_capacity(void);

#ifdef __cplusplus
}
#endif
