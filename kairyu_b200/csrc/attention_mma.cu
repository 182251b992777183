// Exported entry points of the tensor-core attention kernels (attention_mma.cuh).
#include "attention_mma.cuh"

KB_EXPORT int kb_attention_prefill_mma(const void* q, int q_stride, void* out, int out_stride,
                                       const void* k_cache, const void* v_cache,
                                       const int* qo_indptr, const int* seq_lens,
                                       const int* block_table, int max_pages, const int* tile_rows,
                                       const int* tile_starts, int num_tiles, int Hq, int Hkv, int D,
                                       int page_size, int num_pages, float scale, int window, int* flag,
                                       cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if (!q || !out || !k_cache || !v_cache || !qo_indptr || !seq_lens || !block_table || !tile_rows || !tile_starts) return KB_ERR_NULL;
    if (Hkv < 1 || Hq % Hkv != 0 || num_tiles > 65535) return KB_ERR_BAD_ARG;
    if (q_stride % 8 != 0 || out_stride % 2 != 0) return KB_ERR_BAD_ARG;  // 16-byte rows for cp.async
    const int dp = padded_dim(D);
#define ARGS (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_cache, \
             (const __nv_bfloat16*)v_cache, qo_indptr, seq_lens, block_table, max_pages, tile_rows,       \
             tile_starts, num_tiles, Hq, Hkv, D, page_size, num_pages, scale, window, flag, stream
    switch (dp) {
        case 32: return launch_prefill<32, 2>(ARGS);
        case 64: return launch_prefill<64, 2>(ARGS);
        case 128: return launch_prefill<128, 2>(ARGS);
        case 256: return launch_prefill<256, 1>(ARGS);
        default: return KB_ERR_UNSUPPORTED_SIZE;
    }
#undef ARGS
}

// part_o: [rows, Hq, splits, D] fp32; part_ml: [rows, Hq, splits, 2] fp32 (scratch).
KB_EXPORT int kb_attention_decode_mma(const void* q, int q_stride, void* out, int out_stride,
                                      const void* k_cache, const void* v_cache, const int* seq_lens,
                                      const int* block_table, int max_pages, const int* decode_rows,
                                      const int* decode_tokens, int num_rows, int Hq, int Hkv, int D,
                                      int page_size, int num_pages, float scale, int window,
                                      int num_splits, float* part_o, float* part_ml, int* flag,
                                      cudaStream_t stream) {
    if (num_rows == 0) return 0;
    if (!q || !out || !k_cache || !v_cache || !seq_lens || !block_table || !decode_rows || !decode_tokens || !part_o || !part_ml) return KB_ERR_NULL;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16 || Hkv > 65535 || num_splits < 1 || num_splits > 65535) return KB_ERR_BAD_ARG;
    if (q_stride % 8 != 0) return KB_ERR_BAD_ARG;
    const int dp = padded_dim(D);
    int rc;
#define ARGS (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
             seq_lens, block_table, max_pages, decode_rows, decode_tokens, num_rows, Hq, Hkv, D,        \
             page_size, num_pages, scale, window, num_splits, part_o, part_ml, flag, stream
    switch (dp) {
        case 32: rc = launch_decode<32>(ARGS); break;
        case 64: rc = launch_decode<64>(ARGS); break;
        case 128: rc = launch_decode<128>(ARGS); break;
        case 256: rc = launch_decode<256>(ARGS); break;
        default: return KB_ERR_UNSUPPORTED_SIZE;
    }
#undef ARGS
    if (rc != 0) return rc;
    dim3 grid(num_rows, Hq);
    kb_launch(attention_decode_merge_kernel, dim3(grid), dim3(128), 0, stream, part_o, part_ml, seq_lens, decode_rows, decode_tokens,
                                                            (__nv_bfloat16*)out, out_stride, Hq, D, window, num_splits);
    return kb_launch_result();
}

KB_EXPORT int kb_attention_decode_split_size() { return DEC_SPLIT; }

// Queries per tile the prefill kernel expects in its tile list, for a head size.
KB_EXPORT int kb_attention_prefill_tile_rows(int D) { return prefill_tile_rows(D); }
