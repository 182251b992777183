// Per-head RMSNorm of q and k (optional), rotary position encoding, and the
// write of k and v into the paged cache: one pass over the packed qkv rows.
//
//   q, k <- RMSNorm_D(q, k) * w           (kairyu/models/attention.py:162-199, before RoPE)
//   q, k <- u*cos + rotate_half(u)*sin    (kairyu/models/layers.py:165-190)
//   K[slot], V[slot] <- k, v  where slot = table[row, pos / P] * P + pos % P and
//   pos >= write_from[row]               (kairyu/engine/core/kv_pool.py:163-189)
//
// All arithmetic is fp32 with one rounding at the store (the reference's GPU
// kernels round cos, sin and each product to bf16 first, kairyu/kernels/rope_gpu.py:74-112).
#include "common.cuh"

#define ROPE_WARPS 4
#define ROPE_MAX_D 512

template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };
__device__ __forceinline__ float2 pair_to_float(float2 v) { return v; }
__device__ __forceinline__ float2 pair_to_float(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename T> __device__ __forceinline__ typename Pair<T>::type pair_from_float(float a, float b);
template <> __device__ __forceinline__ float2 pair_from_float<float>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from_float<__nv_bfloat16>(float a, float b) { return __floats2bfloat162_rn(a, b); }

// grid (tokens, ceil((Hq + 2*Hkv) / ROPE_WARPS)); one warp per head: q heads, then k
// heads (norm + rotation, k also into the cache), then v heads (copied into the cache).
// PAIRED (the whole head rotates, 2 * rot_half == D, D a multiple of 4, 16-byte aligned rows):
// a lane holds two neighbouring elements of the first half and their partners of the second
// half in registers, so the rotation needs no shared memory and every access is two elements
// wide; the v heads are copied 16 bytes at a time.  The arithmetic is the same either way.
template <typename T, typename TW, bool PAIRED>
__global__ void __launch_bounds__(ROPE_WARPS * 32)
qk_norm_rope_kv_write_kernel(T* __restrict__ qkv, int qkv_stride, int Hq, int Hkv, int D,
                             const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w,
                             float eps, const float* __restrict__ cos_table,
                             const float* __restrict__ sin_table, int rot_half, int max_pos,
                             const int* __restrict__ positions, const int* __restrict__ row_ids,
                             const int* __restrict__ block_table, int max_pages,
                             const int* __restrict__ write_from, T* __restrict__ k_cache,
                             T* __restrict__ v_cache, int page_size, int num_pages, int* flag) {
    pdl_trigger();
    // Positions, row ids, block tables and write_from come from the host's copy of the step, not from
    // the kernel before this one: the look-ups below run ahead of the wait for that kernel's q | k | v.
    __shared__ float head_buf[ROPE_WARPS][ROPE_MAX_D];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * ROPE_WARPS + warp;
    if (head >= Hq + 2 * Hkv) return;
    const int pos = positions[t];
    const int row = row_ids[t];
    T* token = qkv + (size_t)t * qkv_stride;

    const bool rotate = cos_table != nullptr && rot_half > 0;
    if (rotate && (pos < 0 || pos >= max_pos)) {
        if (lane == 0 && flag) atomicOr(flag, KB_FLAG_BAD_POS);
        pdl_wait();
        return;
    }
    const bool is_v = head >= Hq + Hkv;
    const bool is_k = !is_v && head >= Hq;

    // Where this token's k and v go (or nowhere).
    long long slot = -1;
    if ((is_k || is_v) && k_cache != nullptr && pos >= write_from[row]) {
        const int page_index = pos / page_size;
        const int page = page_index < max_pages ? block_table[(size_t)row * max_pages + page_index] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
        } else {
            slot = (long long)page * page_size + (pos % page_size);
        }
    }
    pdl_wait();
    T* x = token + (size_t)head * D;
    if (is_v) {
        if (slot >= 0) {
            T* vdst = v_cache + ((size_t)slot * Hkv + (head - Hq - Hkv)) * D;
            if (PAIRED) {
                constexpr int PER = 16 / sizeof(T);
                for (int i = lane * PER; i < D; i += 32 * PER)
                    *reinterpret_cast<uint4*>(vdst + i) = *reinterpret_cast<const uint4*>(x + i);
            } else {
                for (int i = lane; i < D; i += 32) vdst[i] = x[i];
            }
        }
        return;
    }
    if (PAIRED) {
        using P2 = typename Pair<T>::type;
        constexpr int MAX_J = ROPE_MAX_D / 128;  // a lane's pairs per half
        const int half = D >> 1;
        const TW* w = is_k ? k_norm_w : q_norm_w;
        float2 a[MAX_J], b[MAX_J];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < MAX_J; ++j) {
            const int i = 2 * lane + 64 * j;
            if (i < half) {
                a[j] = pair_to_float(*reinterpret_cast<const P2*>(x + i));
                b[j] = pair_to_float(*reinterpret_cast<const P2*>(x + half + i));
                ss += a[j].x * a[j].x + a[j].y * a[j].y + b[j].x * b[j].x + b[j].y * b[j].y;
            }
        }
        if (w != nullptr) {
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
            for (int j = 0; j < MAX_J; ++j) {
                const int i = 2 * lane + 64 * j;
                if (i < half) {
                    a[j].x = a[j].x * inv * to_float(w[i]);
                    a[j].y = a[j].y * inv * to_float(w[i + 1]);
                    b[j].x = b[j].x * inv * to_float(w[half + i]);
                    b[j].y = b[j].y * inv * to_float(w[half + i + 1]);
                }
            }
        }
        const float* cos_row = cos_table + (size_t)pos * rot_half;
        const float* sin_row = sin_table + (size_t)pos * rot_half;
        T* kdst = (is_k && slot >= 0) ? k_cache + ((size_t)slot * Hkv + (head - Hq)) * D : nullptr;
#pragma unroll
        for (int j = 0; j < MAX_J; ++j) {
            const int i = 2 * lane + 64 * j;
            if (i < half) {
                const float2 c = *reinterpret_cast<const float2*>(cos_row + i);
                const float2 sn = *reinterpret_cast<const float2*>(sin_row + i);
                // rotate_half(u) = cat(-u[half:], u[:half])
                const P2 lo = pair_from_float<T>(a[j].x * c.x - b[j].x * sn.x, a[j].y * c.y - b[j].y * sn.y);
                const P2 hi = pair_from_float<T>(b[j].x * c.x + a[j].x * sn.x, b[j].y * c.y + a[j].y * sn.y);
                *reinterpret_cast<P2*>(x + i) = lo;
                *reinterpret_cast<P2*>(x + half + i) = hi;
                if (kdst) {
                    *reinterpret_cast<P2*>(kdst + i) = lo;
                    *reinterpret_cast<P2*>(kdst + half + i) = hi;
                }
            }
        }
        return;
    }
    float* buf = head_buf[warp];
    const TW* w = is_k ? k_norm_w : q_norm_w;
    float ss = 0.0f;
    for (int i = lane; i < D; i += 32) {
        const float v = to_float(x[i]);
        buf[i] = v;
        ss += v * v;
    }
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        for (int i = lane; i < D; i += 32) buf[i] = buf[i] * inv * to_float(w[i]);
    }
    __syncwarp();
    const float* cos_row = rotate ? cos_table + (size_t)pos * rot_half : nullptr;
    const float* sin_row = rotate ? sin_table + (size_t)pos * rot_half : nullptr;
    T* kdst = (is_k && slot >= 0) ? k_cache + ((size_t)slot * Hkv + (head - Hq)) * D : nullptr;
    for (int i = lane; i < D; i += 32) {
        float out;
        if (rotate && i < 2 * rot_half) {
            const int j = i < rot_half ? i : i - rot_half;
            const float c = cos_row[j];
            const float sn = sin_row[j];
            // rotate_half(u) = cat(-u[half:], u[:half])
            out = i < rot_half ? buf[i] * c - buf[i + rot_half] * sn : buf[i] * c + buf[i - rot_half] * sn;
        } else {
            out = buf[i];
        }
        const T rounded = from_float<T>(out);
        x[i] = rounded;
        if (kdst) kdst[i] = rounded;
    }
}

// The paired path for many tokens and head sizes up to 128: a warp takes one head of TPW
// consecutive tokens and asks for everything it needs of all of them (position, page, the head's
// elements, cos and sin) before it uses any of it, so the round trips to memory overlap instead
// of following one another token by token.  Same arithmetic as the kernel above.
template <typename T, typename TW, int TPW>
__global__ void __launch_bounds__(ROPE_WARPS * 32)
qk_norm_rope_kv_write_many_kernel(T* __restrict__ qkv, int qkv_stride, int Hq, int Hkv, int D,
                                  const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
                                  const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_pos,
                                  const int* __restrict__ positions, const int* __restrict__ row_ids,
                                  const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int num_pages, int tokens,
                                  int* flag) {
    pdl_trigger();
    pdl_wait();
    using P2 = typename Pair<T>::type;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * ROPE_WARPS + warp;
    if (head >= Hq + 2 * Hkv) return;
    const int t0 = blockIdx.x * TPW;
    const bool is_v = head >= Hq + Hkv;
    const bool is_k = !is_v && head >= Hq;
    const int half = D >> 1;
    const int i = 2 * lane;  // this lane's pair of the first half (and its partners half further)
    const bool lane_on = i < half;

    int pos[TPW];
    long long slot[TPW];
    bool ok[TPW];
#pragma unroll
    for (int tt = 0; tt < TPW; ++tt) {
        const int t = t0 + tt;
        ok[tt] = t < tokens;
        pos[tt] = ok[tt] ? positions[t] : 0;
        slot[tt] = -1;
        if (ok[tt] && (pos[tt] < 0 || pos[tt] >= max_pos)) {
            if (lane == 0 && flag) atomicOr(flag, KB_FLAG_BAD_POS);
            ok[tt] = false;
        }
    }
    if ((is_k || is_v) && k_cache != nullptr) {
#pragma unroll
        for (int tt = 0; tt < TPW; ++tt) {
            if (!ok[tt]) continue;
            const int row = row_ids[t0 + tt];
            if (pos[tt] < write_from[row]) continue;
            const int page_index = pos[tt] / page_size;
            const int page = page_index < max_pages ? block_table[(size_t)row * max_pages + page_index] : -1;
            if (page < 0 || page >= num_pages) {
                if (lane == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
            } else {
                slot[tt] = (long long)page * page_size + (pos[tt] % page_size);
            }
        }
    }
    if (is_v) {
        constexpr int PER = 16 / sizeof(T);
        uint4 held[TPW];
        const bool mine = lane * PER < D;  // D <= 128: one 16-byte piece a lane
#pragma unroll
        for (int tt = 0; tt < TPW; ++tt)
            if (mine && slot[tt] >= 0) held[tt] = *reinterpret_cast<const uint4*>(qkv + (size_t)(t0 + tt) * qkv_stride + (size_t)head * D + lane * PER);
#pragma unroll
        for (int tt = 0; tt < TPW; ++tt)
            if (mine && slot[tt] >= 0)
                *reinterpret_cast<uint4*>(v_cache + ((size_t)slot[tt] * Hkv + (head - Hq - Hkv)) * D + lane * PER) = held[tt];
        return;
    }
    float2 a[TPW], b[TPW], c[TPW], sn[TPW];
#pragma unroll
    for (int tt = 0; tt < TPW; ++tt) {
        a[tt] = b[tt] = c[tt] = sn[tt] = make_float2(0.0f, 0.0f);
        if (ok[tt] && lane_on) {
            const T* x = qkv + (size_t)(t0 + tt) * qkv_stride + (size_t)head * D;
            a[tt] = pair_to_float(*reinterpret_cast<const P2*>(x + i));
            b[tt] = pair_to_float(*reinterpret_cast<const P2*>(x + half + i));
            c[tt] = *reinterpret_cast<const float2*>(cos_table + (size_t)pos[tt] * half + i);
            sn[tt] = *reinterpret_cast<const float2*>(sin_table + (size_t)pos[tt] * half + i);
        }
    }
    const TW* w = is_k ? k_norm_w : q_norm_w;
    if (w != nullptr) {
        float2 wa = make_float2(0.0f, 0.0f), wb = wa;
        if (lane_on) {
            wa = make_float2(to_float(w[i]), to_float(w[i + 1]));
            wb = make_float2(to_float(w[half + i]), to_float(w[half + i + 1]));
        }
#pragma unroll
        for (int tt = 0; tt < TPW; ++tt) {
            float ss = a[tt].x * a[tt].x + a[tt].y * a[tt].y + b[tt].x * b[tt].x + b[tt].y * b[tt].y;
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + eps);
            a[tt].x = a[tt].x * inv * wa.x;
            a[tt].y = a[tt].y * inv * wa.y;
            b[tt].x = b[tt].x * inv * wb.x;
            b[tt].y = b[tt].y * inv * wb.y;
        }
    }
#pragma unroll
    for (int tt = 0; tt < TPW; ++tt) {
        if (!ok[tt] || !lane_on) continue;
        T* x = qkv + (size_t)(t0 + tt) * qkv_stride + (size_t)head * D;
        // rotate_half(u) = cat(-u[half:], u[:half])
        const P2 lo = pair_from_float<T>(a[tt].x * c[tt].x - b[tt].x * sn[tt].x, a[tt].y * c[tt].y - b[tt].y * sn[tt].y);
        const P2 hi = pair_from_float<T>(b[tt].x * c[tt].x + a[tt].x * sn[tt].x, b[tt].y * c[tt].y + a[tt].y * sn[tt].y);
        *reinterpret_cast<P2*>(x + i) = lo;
        *reinterpret_cast<P2*>(x + half + i) = hi;
        if (is_k && slot[tt] >= 0) {
            T* kdst = k_cache + ((size_t)slot[tt] * Hkv + (head - Hq)) * D;
            *reinterpret_cast<P2*>(kdst + i) = lo;
            *reinterpret_cast<P2*>(kdst + half + i) = hi;
        }
    }
}

// Many bf16 tokens with heads of 128 or 64 that rotate whole: D / 16 lanes take one head at a time and
// walk a slice of the token's heads, sixteen bytes a lane at a time (eight elements of the first half
// and their partners of the second), so a token's cos and sin rows are fetched once for all its heads
// and every access is 16 bytes wide.  All loads of a lane's heads go out before the first result is
// stored.  Same arithmetic as the kernels above.
#define ROPE_WIDE_TOKENS 4   // tokens a block of 256 threads takes: 64 threads a token
#define ROPE_WIDE_HEADS 8    // heads a group of lanes may be dealt: (Hq + 2 Hkv) <= 8 * (64 / (D / 16))

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

template <typename TW, int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_kv_write_wide_kernel(__nv_bfloat16* __restrict__ qkv, int qkv_stride, int Hq, int Hkv,
                                  const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
                                  const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_pos,
                                  const int* __restrict__ positions, const int* __restrict__ row_ids,
                                  const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                                  __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int page_size,
                                  int num_pages, int tokens, int* flag) {
    pdl_trigger();
    static_assert(D == 128 || D == 64, "heads of 128 or 64");
    constexpr int HALF = D / 2;
    constexpr int LANES = HALF / 8;       // lanes that share a head: 8 elements of each half a lane
    constexpr int SLICES = 64 / LANES;    // groups of lanes a token has
    const int sub = threadIdx.x % LANES;  // this lane's 8 elements of each half
    const int t = blockIdx.x * ROPE_WIDE_TOKENS + (threadIdx.x >> 6);
    const int slice = (threadIdx.x / LANES) % SLICES;  // heads slice, slice + SLICES, ...
    const int heads = Hq + 2 * Hkv;
    // the step's description comes from the host's copy, not from the kernel before: looked up ahead of the wait
    int pos = 0;
    long long slot = -1;
    bool ok = t < tokens;
    if (ok) {
        pos = positions[t];
        if (pos < 0 || pos >= max_pos) {
            if (sub == 0 && slice == 0 && flag) atomicOr(flag, KB_FLAG_BAD_POS);
            ok = false;
        }
    }
    if (ok && k_cache != nullptr) {
        const int row = row_ids[t];
        if (pos >= write_from[row]) {
            const int page_index = pos / page_size;
            const int page = page_index < max_pages ? block_table[(size_t)row * max_pages + page_index] : -1;
            if (page < 0 || page >= num_pages) {
                if (sub == 0 && slice == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
            } else {
                slot = (long long)page * page_size + (pos % page_size);
            }
        }
    }
    float c[8], sn[8];
    if (ok) {
        const float4* cr = reinterpret_cast<const float4*>(cos_table + (size_t)pos * HALF + sub * 8);
        const float4* sr = reinterpret_cast<const float4*>(sin_table + (size_t)pos * HALF + sub * 8);
        const float4 c0 = cr[0], c1 = cr[1], s0 = sr[0], s1 = sr[1];
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    pdl_wait();
    if (!ok) return;
    __nv_bfloat16* token = qkv + (size_t)t * qkv_stride;
    uint4 lo_raw[ROPE_WIDE_HEADS], hi_raw[ROPE_WIDE_HEADS];
#pragma unroll
    for (int n = 0; n < ROPE_WIDE_HEADS; ++n) {
        const int head = slice + SLICES * n;
        if (head < heads) {
            lo_raw[n] = *reinterpret_cast<const uint4*>(token + (size_t)head * D + sub * 8);
            hi_raw[n] = *reinterpret_cast<const uint4*>(token + (size_t)head * D + HALF + sub * 8);
        }
    }
#pragma unroll
    for (int n = 0; n < ROPE_WIDE_HEADS; ++n) {
        const int head = slice + SLICES * n;
        if (head >= heads) break;
        if (head >= Hq + Hkv) {  // a value head: copied as it is
            if (slot >= 0) {
                __nv_bfloat16* vdst = v_cache + ((size_t)slot * Hkv + (head - Hq - Hkv)) * D;
                *reinterpret_cast<uint4*>(vdst + sub * 8) = lo_raw[n];
                *reinterpret_cast<uint4*>(vdst + HALF + sub * 8) = hi_raw[n];
            }
            continue;
        }
        const bool is_k = head >= Hq;
        float a[8], b[8];
        unpack8(lo_raw[n], a);
        unpack8(hi_raw[n], b);
        const TW* w = is_k ? k_norm_w : q_norm_w;
        if (w != nullptr) {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
            // the head's own lanes only: the other groups of the warp may be at other heads, or gone
            const unsigned mates = ((1u << LANES) - 1u) << ((threadIdx.x & 31) & ~(LANES - 1));
#pragma unroll
            for (int step = 1; step < LANES; step <<= 1) ss += __shfl_xor_sync(mates, ss, step);
            const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[i] = a[i] * inv * to_float(w[sub * 8 + i]);
                b[i] = b[i] * inv * to_float(w[HALF + sub * 8 + i]);
            }
        }
        float lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {  // rotate_half(u) = cat(-u[half:], u[:half])
            lo[i] = a[i] * c[i] - b[i] * sn[i];
            hi[i] = b[i] * c[i] + a[i] * sn[i];
        }
        const uint4 lo_out = pack8(lo), hi_out = pack8(hi);
        *reinterpret_cast<uint4*>(token + (size_t)head * D + sub * 8) = lo_out;
        *reinterpret_cast<uint4*>(token + (size_t)head * D + HALF + sub * 8) = hi_out;
        if (is_k && slot >= 0) {
            __nv_bfloat16* kdst = k_cache + ((size_t)slot * Hkv + (head - Hq)) * D;
            *reinterpret_cast<uint4*>(kdst + sub * 8) = lo_out;
            *reinterpret_cast<uint4*>(kdst + HALF + sub * 8) = hi_out;
        }
    }
}

// qkv: [T, qkv_stride] with q | k | v packed per token, head-major.
// *_norm_w: [D] (both or neither), norm_w_bf16 says which type.
// cos/sin: [max_pos, rot_half] fp32 or null.  caches: [num_pages, page_size, Hkv, D] or null.
KB_EXPORT int kb_qk_norm_rope_kv_write(void* qkv, int is_bf16, int T, int qkv_stride, int Hq,
                                       int Hkv, int D, const void* q_norm_w, const void* k_norm_w,
                                       int norm_w_bf16, float eps, const float* cos_table,
                                       const float* sin_table, int rot_half, int max_pos,
                                       const int* positions, const int* row_ids,
                                       const int* block_table, int max_pages,
                                       const int* write_from, void* k_cache, void* v_cache,
                                       int page_size, int num_pages, int* flag,
                                       cudaStream_t stream) {
    if (T == 0) return 0;
    if (!qkv || !positions || !row_ids) return KB_ERR_NULL;
    if (D < 1 || D > ROPE_MAX_D || 2 * rot_half > D) return KB_ERR_UNSUPPORTED_SIZE;
    if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return KB_ERR_BAD_ARG;
    if (k_cache && (!block_table || !write_from || !v_cache || page_size < 1)) return KB_ERR_NULL;
    const int threads = ROPE_WARPS * 32;
    if (Hq + 2 * Hkv > 65535 * ROPE_WARPS) return KB_ERR_UNSUPPORTED_SIZE;
    dim3 grid(T, (Hq + 2 * Hkv + ROPE_WARPS - 1) / ROPE_WARPS);
    // The paired path wants the whole head rotated and every row of qkv and of the caches on a 16-byte boundary.
    const size_t elem = is_bf16 ? 2 : 4;
    const bool paired = cos_table != nullptr && sin_table != nullptr && rot_half > 0 && 2 * rot_half == D && D % 4 == 0 &&
                        (D * elem) % 16 == 0 && ((size_t)qkv_stride * elem) % 16 == 0 && ((uintptr_t)qkv % 16) == 0 &&
                        ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 &&
                        ((uintptr_t)cos_table % 8) == 0 && ((uintptr_t)sin_table % 8) == 0;
    // many bf16 tokens, heads of 128 or 64: 16 bytes a lane, cos and sin fetched once a token
    if (paired && is_bf16 && (D == 128 || D == 64) && T >= 256 && Hq + 2 * Hkv <= (64 / (D / 16)) * ROPE_WIDE_HEADS &&
        ((uintptr_t)cos_table % 16) == 0 && ((uintptr_t)sin_table % 16) == 0) {
        dim3 wide((T + ROPE_WIDE_TOKENS - 1) / ROPE_WIDE_TOKENS);
#define WIDE(TW_, D_)                                                                                          \
    kb_launch(qk_norm_rope_kv_write_wide_kernel<TW_, D_>, dim3(wide), dim3(256), 0, stream, (__nv_bfloat16*)qkv, \
        qkv_stride, Hq, Hkv, (const TW_*)q_norm_w, (const TW_*)k_norm_w, eps, cos_table, sin_table, max_pos,   \
        positions, row_ids, block_table, max_pages, write_from, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, \
        page_size, num_pages, T, flag)
        if (D == 128) {
            if (norm_w_bf16) WIDE(__nv_bfloat16, 128);
            else WIDE(float, 128);
        } else {
            if (norm_w_bf16) WIDE(__nv_bfloat16, 64);
            else WIDE(float, 64);
        }
#undef WIDE
        return kb_launch_result();
    }
    // many tokens, heads of up to 128: four tokens a warp, their memory round trips overlapped
    if (paired && D <= 128 && T >= 256) {
        constexpr int TPW = 4;
        dim3 many((T + TPW - 1) / TPW, (Hq + 2 * Hkv + ROPE_WARPS - 1) / ROPE_WARPS);
#define MANY(T_, TW_)                                                                                   \
    kb_launch(qk_norm_rope_kv_write_many_kernel<T_, TW_, TPW>, dim3(many), dim3(threads), 0, stream,   \
        (T_*)qkv, qkv_stride, Hq, Hkv, D, (const TW_*)q_norm_w, (const TW_*)k_norm_w, eps, cos_table,   \
        sin_table, max_pos, positions, row_ids, block_table, max_pages, write_from, (T_*)k_cache,       \
        (T_*)v_cache, page_size, num_pages, T, flag)
        if (is_bf16) {
            if (norm_w_bf16) MANY(__nv_bfloat16, __nv_bfloat16);
            else MANY(__nv_bfloat16, float);
        } else {
            if (norm_w_bf16) MANY(float, __nv_bfloat16);
            else MANY(float, float);
        }
#undef MANY
        return kb_launch_result();
    }
#define LAUNCH(T_, TW_, P_)                                                                     \
    kb_launch(qk_norm_rope_kv_write_kernel<T_, TW_, P_>, dim3(grid), dim3(threads), 0, stream,  \
        (T_*)qkv, qkv_stride, Hq, Hkv, D, (const TW_*)q_norm_w, (const TW_*)k_norm_w, eps,      \
        cos_table, sin_table, rot_half, max_pos, positions, row_ids, block_table, max_pages,    \
        write_from, (T_*)k_cache, (T_*)v_cache, page_size, num_pages, flag)
#define PICK(T_, TW_) do { if (paired) LAUNCH(T_, TW_, true); else LAUNCH(T_, TW_, false); } while (0)
    if (is_bf16) {
        if (norm_w_bf16) PICK(__nv_bfloat16, __nv_bfloat16);
        else PICK(__nv_bfloat16, float);
    } else {
        if (norm_w_bf16) PICK(float, __nv_bfloat16);
        else PICK(float, float);
    }
#undef PICK
#undef LAUNCH
    return kb_launch_result();
}
