// Token selection on the device: argmax, logit edits (penalties and masks),
// and temperature / min-p / top-k / top-p sampling with a stateless Gumbel-max
// draw (kairyu/engine/core/sampler.py:1198-1389, kairyu/kernels/sampling_gpu.py:51-128).
//
// One block per row.  Every reduction has a fixed order, so a draw is a pure
// function of (logits row, parameters, seed): the same on every run and in
// every batch composition.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)

// ------------------------------------------------------------------ block argmax helpers
struct BestF {
    float v;
    int i;
};

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return v > bv || (v == bv && i < bi);
}

__device__ __forceinline__ BestF block_argmax(BestF b, float* sv, int* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (better(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = b.v; si[warp] = b.i; }
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    BestF r;
    r.v = lane < warps ? sv[lane] : -INFINITY;
    r.i = lane < warps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, r.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, r.i, o);
        if (better(ov, oi, r.v, r.i)) { r.v = ov; r.i = oi; }
    }
    return r;
}

// ------------------------------------------------------------------ argmax
// out[r] = first index of the maximum of logits[r, :] (NaN never wins).
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out, int vectorised) {
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    BestF b{-INFINITY, 0x7fffffff};
    if (vectorised) {  // rows 16-byte aligned: four loads of four in flight per thread
        const int quads = V >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int q0 = threadIdx.x; q0 < quads; q0 += 4 * blockDim.x) {
            float4 part[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * blockDim.x;
                part[u] = q < quads ? row4[q] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = (q0 + u * blockDim.x) * 4;
                if (better(part[u].x, i, b.v, b.i)) { b.v = part[u].x; b.i = i; }
                if (better(part[u].y, i + 1, b.v, b.i)) { b.v = part[u].y; b.i = i + 1; }
                if (better(part[u].z, i + 2, b.v, b.i)) { b.v = part[u].z; b.i = i + 2; }
                if (better(part[u].w, i + 3, b.v, b.i)) { b.v = part[u].w; b.i = i + 3; }
            }
        }
        for (int i = (quads << 2) + threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
    }
    b = block_argmax(b, sv, si);
    if (threadIdx.x == 0) out[blockIdx.x] = b.i == 0x7fffffff ? 0 : b.i;
}

KB_EXPORT int kb_argmax(const float* logits, int ld, int n, int V, int* out, cudaStream_t stream) {
    if (n == 0) return 0;
    if (!logits || !out) return KB_ERR_NULL;
    if (V < 1) return KB_ERR_BAD_ARG;
    const int vectorised = ((uintptr_t)logits % 16 == 0) && (ld % 4 == 0);
    kb_launch(argmax_kernel, dim3(n), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, out, vectorised);
    return kb_launch_result();
}

// ------------------------------------------------------------------ logit edits
// entry e: logits[row[e], tok[e]] <- -inf if mask[e], else
//   l <- (l > 0 ? l / mul[e] : l * mul[e]) - sub[e]
// (repetition penalty over prompt+outputs, frequency*count + presence over
// outputs: kairyu/engine/core/sampler.py:466-502; min-tokens mask: 666-699).
// Entries of one row name distinct tokens, so no two threads touch one logit.
__global__ void edit_logits_kernel(float* __restrict__ logits, int ld, int V,
                                   const int* __restrict__ e_row, const int* __restrict__ e_tok,
                                   const float* __restrict__ e_mul, const float* __restrict__ e_sub,
                                   const int* __restrict__ e_mask, int E) {
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int tok = e_tok[e];
    if (tok < 0 || tok >= V) return;
    float* p = logits + (size_t)e_row[e] * ld + tok;
    if (e_mask[e]) { *p = -INFINITY; return; }
    float l = *p;
    const float mul = e_mul[e];
    if (mul != 1.0f) l = l > 0.0f ? l / mul : l * mul;
    *p = l - e_sub[e];
}

KB_EXPORT int kb_edit_logits(float* logits, int ld, int V, const int* e_row, const int* e_tok,
                             const float* e_mul, const float* e_sub, const int* e_mask, int E,
                             cudaStream_t stream) {
    if (E == 0) return 0;
    if (!logits || !e_row || !e_tok || !e_mul || !e_sub || !e_mask) return KB_ERR_NULL;
    kb_launch(edit_logits_kernel, dim3((E + 255) / 256), dim3(256), 0, stream, logits, ld, V, e_row, e_tok, e_mul, e_sub, e_mask, E);
    return kb_launch_result();
}

// ------------------------------------------------------------------ sampling
__device__ __forceinline__ unsigned long long splitmix_finalize(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Flipped Gumbel noise of vocabulary index i under a per-(request, position) seed.
__device__ __forceinline__ double gumbel_noise(int i, unsigned long long seed) {
    const unsigned long long counter = ((unsigned long long)i + 1ull) * 0x9E3779B97F4A7C15ull;
    const unsigned long long word = splitmix_finalize(counter ^ seed);
    const double u = ((double)(word & ((1ull << 52) - 1ull)) + 0.5) * (1.0 / 4503599627370496.0);
    return -log(-log1p(-u));
}

// Sums 16 per-thread values over the block in a fixed order; result in s_out[16].
__device__ __forceinline__ void block_sum16(float (&local)[16], float (*s_part)[16], float* s_out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 0; d < 16; ++d) local[d] = warp_sum(local[d]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int d = 0; d < 16; ++d) s_part[warp][d] = local[d];
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        float total = 0.0f;
        for (int w = 0; w < SAMPLE_WARPS; ++w) total += s_part[w][threadIdx.x];
        s_out[threadIdx.x] = total;
    }
    __syncthreads();
}

// Smallest 32-bit key u such that weight{ key_i > u, key_i >= lo_key } < target,
// where key_i are the bits of the non-negative floats p_i and weight is a count
// (use_sum = 0) or the sum of p_i (use_sum = 1).  Radix descent, 4 bits a round.
// Requires target > 0.  Every thread returns u.
__device__ unsigned int select_key(const float* __restrict__ p, int V, unsigned int lo_key,
                                   float target, int use_sum, float (*s_part)[16], float* s_out) {
    unsigned int prefix = 0;
    float above = 0.0f;
    for (int shift = 28; shift >= 0; shift -= 4) {
        float local[16];
#pragma unroll
        for (int d = 0; d < 16; ++d) local[d] = 0.0f;
        const unsigned int high_mask = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float pv = p[i];
            const unsigned int key = __float_as_uint(pv);
            if (key < lo_key) continue;
            if ((key & high_mask) != (prefix & high_mask)) continue;
            const int digit = (key >> shift) & 15;
            const float wgt = use_sum ? pv : 1.0f;
#pragma unroll
            for (int d = 0; d < 16; ++d)
                if (d == digit) local[d] += wgt;
        }
        block_sum16(local, s_part, s_out);
        // G(d) = above + sum_{e>d} S[e]; pick the smallest d with G(d) < target.
        int d = 15;
        float g = above;  // G(15)
        while (d > 0) {
            const float g_next = g + s_out[d];  // G(d-1)
            if (!(g_next < target)) break;
            g = g_next;
            --d;
        }
        above = g;
        prefix |= (unsigned int)d << shift;
        __syncthreads();  // s_out is rewritten next round
    }
    return prefix;
}

// logits: [n, V] fp32 (read only); work: [n, V] fp32 scratch (probabilities).
// Per row: temperature (0 = argmax), top_k (<=0 or >=V: off), top_p (>=1: off),
// min_p (<=0: off), seed (already mixed with the output position).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, float* __restrict__ work, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const unsigned long long* __restrict__ seeds, int* __restrict__ out) {
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float s_part[SAMPLE_WARPS][16];
    __shared__ float s_out[16];
    __shared__ double dv[32];
    __shared__ int di[32];

    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature[r];

    if (T == 0.0f) {
        BestF b{-INFINITY, 0x7fffffff};
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
        b = block_argmax(b, sv, si);
        if (threadIdx.x == 0) out[r] = b.i == 0x7fffffff ? 0 : b.i;
        return;
    }

    float* p = work + (size_t)r * V;
    // softmax(logits / T)
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] / T);
    mx = block_max(mx, scratch);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) sum += expf(row[i] / T - mx);
    sum = block_sum(sum, scratch);
    // min-p: keep p >= min_p * max p (sampler.py:1244-1249)
    const float mp = min_p[r];
    const float p_max = 1.0f / sum;  // exp(0) / sum
    const float floor_p = mp > 0.0f ? mp * p_max : 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float pv = expf(row[i] / T - mx) / sum;
        if (pv < floor_p) pv = 0.0f;
        p[i] = pv;
    }
    __syncthreads();

    unsigned int lo_key = 0;
    // top-k: keep p >= k-th largest (ties kept) (sampler.py:1259-1291)
    const int k = top_k[r];
    if (k > 0 && k < V) lo_key = select_key(p, V, lo_key, (float)k, 0, s_part, s_out);
    // top-p: in descending order drop a token once the mass before it reaches
    // top_p * total (sampler.py:1349-1361); tokens tied with the last kept one stay.
    const float tp = top_p[r];
    if (tp < 1.0f) {
        float total = 0.0f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float pv = p[i];
            if (__float_as_uint(pv) >= lo_key) total += pv;
        }
        total = block_sum(total, scratch);
        const float target = tp * fmaxf(total, 1e-12f);
        const unsigned int u = select_key(p, V, lo_key, target, 1, s_part, s_out);
        lo_key = u > lo_key ? u : lo_key;
    }
    // renormalise over what is left, add the noise, take the argmax
    float kept = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float pv = p[i];
        if (pv > 0.0f && __float_as_uint(pv) >= lo_key) kept += pv;
    }
    kept = block_sum(kept, scratch);
    if (!(kept > 0.0f)) {  // everything filtered: fall back to the argmax (sampler.py:1363-1378)
        BestF b{-INFINITY, 0x7fffffff};
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
        b = block_argmax(b, sv, si);
        if (threadIdx.x == 0) out[r] = b.i == 0x7fffffff ? 0 : b.i;
        return;
    }
    const unsigned long long seed = seeds[r];
    double best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float pv = p[i];
        if (pv > 0.0f && __float_as_uint(pv) >= lo_key) {
            const double v = (double)logf(pv / kept) + gumbel_noise(i, seed);
            if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
        }
    }
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const double ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { dv[warp] = best; di[warp] = best_i; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < SAMPLE_WARPS; ++w)
                if (dv[w] > best || (dv[w] == best && di[w] < best_i)) { best = dv[w]; best_i = di[w]; }
            out[r] = best_i == 0x7fffffff ? 0 : best_i;
        }
    }
}

KB_EXPORT int kb_sample(const float* logits, int ld, float* work, int n, int V,
                        const float* temperature, const int* top_k, const float* top_p,
                        const float* min_p, const unsigned long long* seeds, int* out,
                        cudaStream_t stream) {
    if (n == 0) return 0;
    if (!logits || !work || !temperature || !top_k || !top_p || !min_p || !seeds || !out) return KB_ERR_NULL;
    if (V < 1 || V >= (1 << 24)) return KB_ERR_UNSUPPORTED_SIZE;  // counts are kept in fp32
    kb_launch(sample_kernel, dim3(n), dim3(SAMPLE_THREADS), 0, stream, logits, ld, work, V, temperature, top_k, top_p, min_p, seeds, out);
    return kb_launch_result();
}
