// Paged GQA attention, one block per (query token, query head), fp32 arithmetic
// throughout.  This is the 32-bit path's attention and the fallback for sizes
// the tensor-core kernels refuse.
//
// Query at absolute position p of request row r sees keys j with
// max(0, p + 1 - window) <= j <= p (kairyu/engine/core/attention/torch_backend.py:57-71;
// the window is this engine's addition for cache groups that keep only recent keys).
// Query head h reads KV head h / (Hq / Hkv).  S = q.k * scale, softmax, P.V.
//
// The order of every sum depends only on (p, window, D): warp w of the block
// takes keys start+w, start+w+4, ... with an online softmax of its own, and the
// four partial results are merged in warp order.  So a token's output does not
// depend on what else is in the batch or how the prompt was cut.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_D 256
#define ATT_MAX_K (ATT_MAX_D / 32)

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                               int out_stride, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ positions,
                               const int* __restrict__ row_ids,
                               const int* __restrict__ block_table, int max_pages, int Hq, int Hkv,
                               int D, int page_size, int num_pages, float scale, int window,
                               int* flag) {
    pdl_wait();
    __shared__ float sm_acc[ATT_WARPS][ATT_MAX_D];
    __shared__ float sm_m[ATT_WARPS];
    __shared__ float sm_l[ATT_WARPS];

    const int t = blockIdx.x;
    const int h = blockIdx.y;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int row = row_ids[t];
    const int kvh = h / (Hq / Hkv);
    const int* table = block_table + (size_t)row * max_pages;
    const int start = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;

    float qv[ATT_MAX_K];
    const T* qp = q + (size_t)t * q_stride + (size_t)h * D;
#pragma unroll
    for (int k = 0; k < ATT_MAX_K; ++k) {
        const int e = lane + 32 * k;
        qv[k] = e < D ? to_float(qp[e]) : 0.0f;
    }

    float m = -INFINITY, l = 0.0f;
    float acc[ATT_MAX_K];
#pragma unroll
    for (int k = 0; k < ATT_MAX_K; ++k) acc[k] = 0.0f;

    for (int j = start + warp; j <= pos; j += ATT_WARPS) {
        const int page_index = j / page_size;
        int page = page_index < max_pages ? table[page_index] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
            continue;
        }
        const size_t base = (((size_t)page * page_size + (j % page_size)) * Hkv + kvh) * D;
        const T* kp = k_cache + base;
        const T* vp = v_cache + base;
        float dot = 0.0f;
#pragma unroll
        for (int k = 0; k < ATT_MAX_K; ++k) {
            const int e = lane + 32 * k;
            if (e < D) dot += qv[k] * to_float(kp[e]);
        }
        dot = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, dot);
        const float alpha = expf(m - m_new);
        const float p = expf(dot - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int k = 0; k < ATT_MAX_K; ++k) {
            const int e = lane + 32 * k;
            if (e < D) acc[k] = acc[k] * alpha + p * to_float(vp[e]);
        }
        m = m_new;
    }

#pragma unroll
    for (int k = 0; k < ATT_MAX_K; ++k) {
        const int e = lane + 32 * k;
        if (e < D) sm_acc[warp][e] = acc[k];
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
    __syncthreads();

    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) big = fmaxf(big, sm_m[w]);
    float weights[ATT_WARPS];
    float denom = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        weights[w] = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - big);
        denom += sm_l[w] * weights[w];
    }
    T* op = out + (size_t)t * out_stride + (size_t)h * D;
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) v += sm_acc[w][e] * weights[w];
        op[e] = from_float<T>(denom > 0.0f ? v / denom : 0.0f);
    }
}

KB_EXPORT int kb_paged_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                         const void* k_cache, const void* v_cache, int is_bf16,
                                         const int* positions, const int* row_ids,
                                         const int* block_table, int max_pages, int T, int Hq,
                                         int Hkv, int D, int page_size, int num_pages, float scale,
                                         int window, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!q || !out || !k_cache || !v_cache || !positions || !row_ids || !block_table) return KB_ERR_NULL;
    if (D < 1 || D > ATT_MAX_D) return KB_ERR_UNSUPPORTED_SIZE;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq > 65535) return KB_ERR_BAD_ARG;
    dim3 grid(T, Hq);
    if (is_bf16)
        kb_launch(paged_attention_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(ATT_WARPS * 32), 0, stream, 
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
            (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions, row_ids,
            block_table, max_pages, Hq, Hkv, D, page_size, num_pages, scale, window, flag);
    else
        kb_launch(paged_attention_generic_kernel<float>, dim3(grid), dim3(ATT_WARPS * 32), 0, stream, 
            (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_cache,
            (const float*)v_cache, positions, row_ids, block_table, max_pages, Hq, Hkv, D,
            page_size, num_pages, scale, window, flag);
    return kb_launch_result();
}
