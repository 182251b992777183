// Split-KV decode attention with its scratch inside the library (see
// attention_decode_static.h for who needs this and what the limits are).
#include "attention_decode_static.h"

#include "attention_mma.cuh"

#include <cstdint>

#define KB_MAX_DEVICES 64

// The per-split partials of one call: first the unnormalised outputs
// [rows, Hq, splits, D], then (max, sum) pairs [rows, Hq, splits, 2].
static __device__ __align__(256) float kb_decode_scratch[KB_STATIC_SCRATCH_FLOATS];

// In host code `kb_decode_scratch` is only a handle for the runtime, not an
// address a kernel can use: the device address is looked up once per device.
static float* g_scratch_address[KB_MAX_DEVICES];

static int scratch_for_current_device(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= KB_MAX_DEVICES) return KB_ERR_SETUP_FAILED;
    if (g_scratch_address[device] == nullptr) {
        void* found = nullptr;
        e = cudaGetSymbolAddress(&found, kb_decode_scratch);
        if (e != cudaSuccess) return (int)e;
        if (found == nullptr) return KB_ERR_SETUP_FAILED;
        g_scratch_address[device] = static_cast<float*>(found);
    }
    *address = g_scratch_address[device];
    return 0;
}

KB_EXPORT int kb_attention_decode_static_capacity(void) { return KB_STATIC_SCRATCH_FLOATS; }

KB_EXPORT int kb_attention_decode_mma_static(const void* q, int q_stride, void* out, int out_stride,
                                             const void* k_cache, const void* v_cache,
                                             const int* seq_lens, const int* block_table,
                                             int max_pages, const int* decode_rows,
                                             const int* decode_tokens, int num_rows, int Hq, int Hkv,
                                             int D, int page_size, int num_pages, float scale,
                                             int window, int max_seq_len, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    if (!q || !out || !k_cache || !v_cache || !seq_lens || !block_table || !decode_rows || !decode_tokens) return KB_ERR_NULL;
    if (num_rows < 0 || max_seq_len < 1 || Hkv < 1 || Hq < 1 || Hq % Hkv != 0 || Hq / Hkv > 16 || Hkv > 65535) return KB_ERR_BAD_ARG;
    // What the Python wrapper of the ordinary entry point checks on tensors, a C caller has to
    // be told here: the kernel copies 16 bytes at a time from q and from the cache pages.
    if (q_stride % 8 != 0 || q_stride < Hq * D || out_stride < Hq * D) return KB_ERR_BAD_ARG;
    if (page_size < 1 || max_pages < 1 || num_pages < 1 || window < 0 || D < 1) return KB_ERR_BAD_ARG;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 != 0) return KB_ERR_BAD_ARG;
    if ((uintptr_t)out % 2 != 0 || ((uintptr_t)seq_lens | (uintptr_t)block_table | (uintptr_t)decode_rows | (uintptr_t)decode_tokens) % 4 != 0) return KB_ERR_BAD_ARG;
    const int dp = padded_dim(D);
    if (dp == 0) return KB_ERR_UNSUPPORTED_SIZE;
    const long long num_splits = ((long long)max_seq_len + DEC_SPLIT - 1) / DEC_SPLIT;
    if (num_splits > 65535) return KB_ERR_BAD_ARG;
    const long long entries = (long long)num_rows * Hq * num_splits;
    if (entries * (D + 2) > (long long)KB_STATIC_SCRATCH_FLOATS) return KB_ERR_SCRATCH_TOO_SMALL;

    float* scratch = nullptr;
    const int setup = scratch_for_current_device(&scratch);
    if (setup != 0) return setup;
    float* part_o = scratch;
    float* part_ml = scratch + entries * D;

    int rc;
#define ARGS (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
             seq_lens, block_table, max_pages, decode_rows, decode_tokens, num_rows, Hq, Hkv, D,        \
             page_size, num_pages, scale, window, (int)num_splits, part_o, part_ml, (int*)nullptr, stream
    switch (dp) {
        case 32: rc = launch_decode<32>(ARGS); break;
        case 64: rc = launch_decode<64>(ARGS); break;
        case 128: rc = launch_decode<128>(ARGS); break;
        default: rc = launch_decode<256>(ARGS); break;
    }
#undef ARGS
    if (rc != 0) return rc;
    dim3 grid(num_rows, Hq);
    kb_launch(attention_decode_merge_kernel, dim3(grid), dim3(128), 0, stream, part_o, part_ml, seq_lens, decode_rows, decode_tokens,
                                                            (__nv_bfloat16*)out, out_stride, Hq, D, window,
                                                            (int)num_splits);
    return kb_launch_result();
}
