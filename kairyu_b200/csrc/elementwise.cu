// Embedding gather, RMSNorm (with the residual sum fused in) and SiLU-gated
// multiply.  Statistics and the residual sum are 32-bit in every variant.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :] as fp32 (the residual stream is fp32 in both
// modes).  An id outside [0, V) writes zeros and raises KB_FLAG_BAD_TOKEN.
template <typename TT>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int H, int V, int* flag) {
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    const TT* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_float(src[i]);
}

KB_EXPORT int kb_embedding(const void* table, int table_is_bf16, const int* ids, float* out, int T,
                           int H, int V, int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!table || !ids || !out) return KB_ERR_NULL;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_is_bf16)
        kb_launch(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, out, H, V, flag);
    else
        kb_launch(embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, out, H, V, flag);
    return kb_launch_result();
}

// ------------------------------------------------------------------ tokens that are still on the device
// ids[t] = sampled[source[t]] where source[t] >= 0: the token a step is fed may be the one the
// step before it has just chosen, which the host has not seen yet
// (kairyu/engine/core/model_runner.py:1998-2041, 2080-2162: device-resident future tokens).
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source,
                                    const int* __restrict__ sampled, int T, int sampled_len, int* flag) {
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int s = source[t];
    if (s < 0) return;
    if (s >= sampled_len) {
        if (flag) atomicOr(flag, KB_FLAG_BAD_ROW);
        return;
    }
    ids[t] = sampled[s];
}

KB_EXPORT int kb_patch_tokens(int* ids, const int* source, const int* sampled, int T, int sampled_len, int* flag,
                              cudaStream_t stream) {
    if (T == 0) return 0;
    if (!ids || !source || !sampled) return KB_ERR_NULL;
    kb_launch(patch_tokens_kernel, dim3((T + 127) / 128), dim3(128), 0, stream, ids, source, sampled, T, sampled_len, flag);
    return kb_launch_result();
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row r; source row s = rows ? rows[r] : r.
//   v = x[s] (+ delta[s]);  if write_back: x[s] = v  (the fp32 residual sum)
//   out[r] = v * rsqrt(mean(v^2) + eps) * w          (kairyu/models/layers.py:42-46,
// without its intermediate rounding of the normalised value: one rounding at the end).
template <typename TX, typename TA, typename TW>
__global__ void rmsnorm_kernel(TX* __restrict__ x, const TA* __restrict__ delta,
                               const TW* __restrict__ w, TA* __restrict__ out,
                               const int* __restrict__ rows, int H, float eps, int write_back) {
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    TX* xr = x + (size_t)s * H;
    const TA* dr = delta ? delta + (size_t)s * H : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_float(xr[i]);
        if (dr) {
            v += to_float(dr[i]);
            if (write_back) xr[i] = from_float<TX>(v);
        }
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    TA* orow = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_float(xr[i]);
        if (dr && !write_back) v += to_float(dr[i]);
        orow[i] = from_float<TA>(v * inv * to_float(w[i]));
    }
}


// Vector variant for H % 4 == 0 and H <= 16 * blockDim: each thread keeps up to four
// 4-element chunks of the row in registers, so the row is read once, all loads are in
// flight together, and one block-wide sum separates the two halves.
#define NORM_MAX_CHUNKS 4

template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <>
struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
        __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 r;
        r.x = *reinterpret_cast<uint32_t*>(&a);
        r.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

// The sum of a row's squares is added in one order whatever the block's size: chunk by chunk (four
// elements each), then group g = 0..G-1 adds the partial sums of chunks g, g + G, g + 2G, g + 3G in that
// order (G = `groups`: the thread count of the block that holds every chunk a thread may), then the groups'
// sums go through block_sum as the values of threads 0..G-1.  A block of G threads has all of a group's
// chunks in one thread; a larger block (a few rows: every load in flight at once) passes the chunks' sums
// through shared memory.  Either way a row's result depends on its width alone.
template <typename TX, typename TA, typename TW>
__global__ void rmsnorm_vec_kernel(TX* __restrict__ x, const TA* __restrict__ delta,
                                   const TW* __restrict__ w, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int write_back, int groups) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float chunk_sums[NORM_MAX_CHUNKS * 1024];
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    TX* xr = x + (size_t)s * H;
    const TA* dr = delta ? delta + (size_t)s * H : nullptr;
    const int chunks = H >> 2;
    float v[NORM_MAX_CHUNKS][4];
    float part[NORM_MAX_CHUNKS];
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
        const int chunk = threadIdx.x + c * blockDim.x;
        part[c] = 0.0f;
        if (chunk < chunks) {
            Vec4<TX>::load(xr + 4 * chunk, v[c]);
            if (dr) {
                float d[4];
                Vec4<TA>::load(dr + 4 * chunk, d);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[c][e] += d[e];
                if (write_back) Vec4<TX>::store(xr + 4 * chunk, v[c]);
            }
            part[c] = ((v[c][0] * v[c][0] + v[c][1] * v[c][1]) + v[c][2] * v[c][2]) + v[c][3] * v[c][3];
        }
    }
    float ss = 0.0f;
    if ((int)blockDim.x == groups) {
#pragma unroll
        for (int c = 0; c < NORM_MAX_CHUNKS; ++c) ss += part[c];  // chunks t, t + G, t + 2G, t + 3G: this thread's own
    } else {
#pragma unroll
        for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
            const int chunk = threadIdx.x + c * blockDim.x;
            if (chunk < NORM_MAX_CHUNKS * 1024) chunk_sums[chunk] = part[c];
        }
        __syncthreads();
        if ((int)threadIdx.x < groups) {
#pragma unroll
            for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
                const int chunk = threadIdx.x + c * groups;
                ss += chunk < chunks ? chunk_sums[chunk] : 0.0f;
            }
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    TA* orow = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
        const int chunk = threadIdx.x + c * blockDim.x;
        if (chunk < chunks) {
            float wv[4], o[4];
            Vec4<TW>::load(w + 4 * chunk, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = v[c][e] * inv * wv[e];
            Vec4<TA>::store(orow + 4 * chunk, o);
        }
    }
}

template <typename TX, typename TA>
static int rmsnorm_dispatch_w(void* x, const void* delta, const void* w, int w_bf16, void* out,
                              const int* rows, int R, int H, float eps, int write_back,
                              cudaStream_t stream) {
    const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                         (delta == nullptr || (uintptr_t)delta % 16 == 0);
    if (H % 4 == 0 && H <= 16 * 1024 && aligned) {
        // Many rows (a prompt portion): blocks that hold every chunk a thread may, so that an SM has eight
        // small blocks in different phases (loads, the sum, stores) instead of two large ones in step (2,048
        // rows of 4,096: 21.5 -> 18.1 us; 8,192 rows: 75 -> 63 us).  A few rows (decode): a chunk a thread,
        // every load in flight at once (in a decode step of 16 rows the small blocks cost 2 us a norm).
        int groups = ((H / 4 + NORM_MAX_CHUNKS - 1) / NORM_MAX_CHUNKS + 31) / 32 * 32;
        if (groups < 128) groups = 128;
        if (groups > 1024) groups = 1024;
        int threads_v = groups;
        if (R < 256) {
            threads_v = ((H / 4 + 31) / 32) * 32;
            if (threads_v > 1024) threads_v = 1024;
            if (threads_v < groups) threads_v = groups;
        }
        if (w_bf16)
            kb_launch(rmsnorm_vec_kernel<TX, TA, __nv_bfloat16>, dim3(R), dim3(threads_v), 0, stream, 
                (TX*)x, (const TA*)delta, (const __nv_bfloat16*)w, (TA*)out, rows, H, eps, write_back, groups);
        else
            kb_launch(rmsnorm_vec_kernel<TX, TA, float>, dim3(R), dim3(threads_v), 0, stream, 
                (TX*)x, (const TA*)delta, (const float*)w, (TA*)out, rows, H, eps, write_back, groups);
        return kb_launch_result();
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (w_bf16)
        kb_launch(rmsnorm_kernel<TX, TA, __nv_bfloat16>, dim3(R), dim3(threads), 0, stream, 
            (TX*)x, (const TA*)delta, (const __nv_bfloat16*)w, (TA*)out, rows, H, eps, write_back);
    else
        kb_launch(rmsnorm_kernel<TX, TA, float>, dim3(R), dim3(threads), 0, stream, 
            (TX*)x, (const TA*)delta, (const float*)w, (TA*)out, rows, H, eps, write_back);
    return kb_launch_result();
}

// x: [*, H] fp32 or bf16 (x_bf16); delta/out: activation dtype (act_bf16); w: fp32 or bf16.
KB_EXPORT int kb_rmsnorm(void* x, int x_bf16, const void* delta, const void* w, int w_bf16,
                         void* out, int act_bf16, const int* rows, int R, int H, float eps,
                         int write_back, cudaStream_t stream) {
    if (R == 0) return 0;
    if (!x || !w || !out) return KB_ERR_NULL;
    if (H < 1) return KB_ERR_BAD_ARG;
    if (rows) write_back = 0;
    if (x_bf16) {
        if (act_bf16)
            return rmsnorm_dispatch_w<__nv_bfloat16, __nv_bfloat16>(x, delta, w, w_bf16, out, rows, R, H, eps, write_back, stream);
        return KB_ERR_BAD_ARG;  // bf16 input with fp32 activations is not a mode of this engine
    }
    if (act_bf16)
        return rmsnorm_dispatch_w<float, __nv_bfloat16>(x, delta, w, w_bf16, out, rows, R, H, eps, write_back, stream);
    return rmsnorm_dispatch_w<float, float>(x, delta, w, w_bf16, out, rows, R, H, eps, write_back, stream);
}

// ------------------------------------------------------------------ SiLU(gate) * up
// gate_up: [T, 2*I] with the gate in columns [0, I) and up in [I, 2I)
// (kairyu/models/layers.py:244); out: [T, I].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I) {
    pdl_wait();
    const int t = blockIdx.y;
    const T* g = gate_up + (size_t)t * 2 * I;
    const T* u = g + I;
    T* o = out + (size_t)t * I;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I; i += gridDim.x * blockDim.x) {
        const float gv = to_float(g[i]);
        const float uv = to_float(u[i]);
        o[i] = from_float<T>(gv / (1.0f + expf(-gv)) * uv);
    }
}


// 8 elements a thread (16-byte loads for bf16, two for fp32) when I % 8 == 0.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I) {
    pdl_wait();
    const int t = blockIdx.y;
    const T* g = gate_up + (size_t)t * 2 * I;
    const T* u = g + I;
    T* o = out + (size_t)t * I;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8; i < I; i += gridDim.x * blockDim.x * 8) {
        float gv[8], uv[8], ov[8];
        Vec4<T>::load(g + i, *reinterpret_cast<float(*)[4]>(&gv[0]));
        Vec4<T>::load(g + i + 4, *reinterpret_cast<float(*)[4]>(&gv[4]));
        Vec4<T>::load(u + i, *reinterpret_cast<float(*)[4]>(&uv[0]));
        Vec4<T>::load(u + i + 4, *reinterpret_cast<float(*)[4]>(&uv[4]));
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            // bf16 rows: the exponential and the quotient by their fast forms (2 ulp of fp32, far below the
            // rounding of the result to bf16; a third of the instructions); fp32 rows: the exact ones
            if (sizeof(T) == 2)
                ov[e] = __fdividef(gv[e], 1.0f + __expf(-gv[e])) * uv[e];
            else
                ov[e] = gv[e] / (1.0f + expf(-gv[e])) * uv[e];
        }
        Vec4<T>::store(o + i, *reinterpret_cast<float(*)[4]>(&ov[0]));
        Vec4<T>::store(o + i + 4, *reinterpret_cast<float(*)[4]>(&ov[4]));
    }
}

KB_EXPORT int kb_swiglu(const void* gate_up, void* out, int is_bf16, int T, int I, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!gate_up || !out) return KB_ERR_NULL;
    if (T > 65535) return KB_ERR_UNSUPPORTED_SIZE;
    const int threads = 256;
    if (I % 8 == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)out % 16 == 0) {
        int bxv = (I / 8 + threads - 1) / threads;
        if (bxv > 1024) bxv = 1024;
        dim3 gridv(bxv, T);
        if (is_bf16)
            kb_launch(swiglu_vec_kernel<__nv_bfloat16>, dim3(gridv), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I);
        else
            kb_launch(swiglu_vec_kernel<float>, dim3(gridv), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I);
        return kb_launch_result();
    }
    int bx = (I + threads - 1) / threads;
    if (bx > 1024) bx = 1024;
    dim3 grid(bx, T);
    if (is_bf16)
        kb_launch(swiglu_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I);
    else
        kb_launch(swiglu_kernel<float>, dim3(grid), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I);
    return kb_launch_result();
}

// ------------------------------------------------------------------ row gather (fp32 or bf16 rows)
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows,
                                   T* __restrict__ out, int H) {
    pdl_wait();
    const T* s = src + (size_t)rows[blockIdx.x] * H;
    T* o = out + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = s[i];
}

KB_EXPORT int kb_gather_rows(const void* src, const int* rows, void* out, int is_bf16, int R, int H,
                             cudaStream_t stream) {
    if (R == 0) return 0;
    if (!src || !rows || !out) return KB_ERR_NULL;
    if (is_bf16)
        kb_launch(gather_rows_kernel<__nv_bfloat16>, dim3(R), dim3(256), 0, stream, (const __nv_bfloat16*)src, rows, (__nv_bfloat16*)out, H);
    else
        kb_launch(gather_rows_kernel<float>, dim3(R), dim3(256), 0, stream, (const float*)src, rows, (float*)out, H);
    return kb_launch_result();
}
