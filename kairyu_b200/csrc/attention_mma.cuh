// (kernels and launchers; attention_mma.cu and attention_decode_static.cu export entry points over them)
// bf16 paged GQA attention on tensor cores (mma.sync m16n8k16, fp32 softmax and
// accumulation): a flash-attention kernel over 64-query tiles for rows that
// carry several tokens, and a split-KV kernel plus a merge for rows that carry
// one token.  Keys and values are read through the block table, 64 keys at a
// time, with cp.async double buffering.
//
// Semantics (kairyu/engine/core/attention/torch_backend.py:57-71): the query at
// absolute position p sees keys max(0, p+1-window) <= j <= p; query head h reads
// KV head h / (Hq/Hkv); S = q.k * scale; softmax over keys; P.V.
//
// Head sizes: any multiple of 16 up to 256; the kernels are instantiated for a
// padded size DP in {32, 64, 128, 256} and zero-fill the columns above D.
// Partition boundaries of the split-KV kernel are absolute key positions
// (multiples of DEC_SPLIT), so a row's result depends only on its own length.
#pragma once
#include "common.cuh"

#define TILE_N 64
#define MMA_THREADS 128
#define DEC_SPLIT 128  // keys per split of the split-KV kernel
#define DEC_STAGES 2  // tile buffers of the split-KV kernel: a split's tiles are all requested up front
#define LOG2E 1.4426950408889634f

// Rows of a shared tile are DP + 8 elements apart: the 16 extra bytes put eight
// consecutive rows in distinct bank groups, so ldmatrix is conflict-free.
template <int DP>
struct Tile {
    static constexpr int STRIDE = DP + 8;
    static constexpr int CHUNKS = DP / 8;  // 16-byte chunks per row
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16-byte async copy; when !valid the destination is zero-filled and the source not read.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }


// ---- mbarrier + bulk copy (the TMA unit moves whole key rows; one instruction per row)
#define KB_FLAG_TIMEOUT 16

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity to complete; gives up when the time limit
// (KB_WAIT_LIMIT_NS) has passed and returns false (the caller raises a flag and leaves).
// `polls` > 0 bounds the wait by that many polls instead: the brief waits of a block that is
// leaving and only lets its copies in flight land.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t polls = 0) {
    const uint32_t addr = smem_u32(bar);
    unsigned long long deadline = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (polls) {
            if (spin + 1 >= polls) return false;
        } else if ((spin & 63) == 63) {
            const unsigned long long now = global_timer_ns();
            if (deadline == 0) deadline = now + KB_WAIT_LIMIT_NS;
            else if (now > deadline) return false;
        }
    }
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
// global -> shared, `bytes` a multiple of 16, both addresses 16-byte aligned; completion is
// counted on the mbarrier.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// One bulk copy per key row: thread t < 64 brings key row t of the K tile, thread
// 64 + t the same row of the V tile.  A row that is outside [key_lo, key_end) or on an
// absent page is read from position 0 of the reserved page instead: its score is masked,
// and what stands there is finite, so the byte count of a tile is always the same.
template <int DP>
__device__ __forceinline__ void load_kv_rows_bulk(__nv_bfloat16* tile_k, __nv_bfloat16* tile_v,
                                                  const __nv_bfloat16* __restrict__ k_cache,
                                                  const __nv_bfloat16* __restrict__ v_cache,
                                                  const int* __restrict__ table, int max_pages, int num_pages,
                                                  int page_size, int page_shift, int Hkv, int kvh, int D,
                                                  int key0, int key_lo, int key_end, uint64_t* bar) {
    if (threadIdx.x == 0) mbar_arrive_expect_tx(bar, (uint32_t)(2 * TILE_N * D * sizeof(__nv_bfloat16)));
    const int r = threadIdx.x & (TILE_N - 1);
    const bool is_v = threadIdx.x >= TILE_N;
    const int key = key0 + r;
    size_t offset = (size_t)kvh * D;  // page 0, position 0
    if (key >= key_lo && key < key_end) {
        const int page_index = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
        const int page = page_index < max_pages ? table[page_index] : -1;
        if (page >= 0 && page < num_pages) {
            const int within = key - page_index * page_size;
            offset = (((size_t)page * page_size + within) * Hkv + kvh) * D;
        }
    }
    bulk_copy_g2s((is_v ? tile_v : tile_k) + r * Tile<DP>::STRIDE, (is_v ? v_cache : k_cache) + offset,
                  (uint32_t)(D * sizeof(__nv_bfloat16)), bar);
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
// d += a(16x16, row) * b(16x8, col), bf16 inputs, fp32 accumulate
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}


// Copies the 64 keys and values starting at absolute key `key0` of one KV head into
// a K tile and a V tile (row r of a tile = key key0 + r).  Keys outside
// [key_lo, key_end), keys on pages the table marks absent, and columns >= D are
// zero-filled.  A thread owns one 16-byte column of the rows r0, r0 + RPP, ...: the
// page lookup is done once per row and shared by the K and the V copy.
template <int DP>
__device__ __forceinline__ void load_kv_tiles(__nv_bfloat16* tile_k, __nv_bfloat16* tile_v,
                                              const __nv_bfloat16* __restrict__ k_cache,
                                              const __nv_bfloat16* __restrict__ v_cache,
                                              const int* __restrict__ table, int max_pages, int num_pages,
                                              int page_size, int page_shift, int Hkv, int kvh, int D,
                                              int key0, int key_lo, int key_end) {
    constexpr int CH = Tile<DP>::CHUNKS;
    constexpr int RPP = MMA_THREADS / CH;  // rows per pass
    constexpr int PASSES = TILE_N / RPP;
    const int col = (threadIdx.x % CH) * 8;
    const int r0 = threadIdx.x / CH;
    const bool col_ok = col < D;
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
        const int r = r0 + pass * RPP;
        const int key = key0 + r;
        bool valid = col_ok && key >= key_lo && key < key_end;
        size_t offset = 0;
        if (valid) {
            const int page_index = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
            const int page = page_index < max_pages ? table[page_index] : -1;
            if (page < 0 || page >= num_pages) {
                valid = false;
            } else {
                const int within = key - page_index * page_size;
                offset = (((size_t)page * page_size + within) * Hkv + kvh) * D + col;
            }
        }
        cp_async16(tile_k + r * Tile<DP>::STRIDE + col, k_cache + offset, valid);
        cp_async16(tile_v + r * Tile<DP>::STRIDE + col, v_cache + offset, valid);
    }
}

__device__ __forceinline__ int shift_of(int page_size) {
    return (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
}

// ------------------------------------------------------------------ prefill: query tiles
// grid (Hq, tiles).  A tile is 64*MT consecutive queries of one row's portion (MT = 2 up to
// a padded head size of 128, else 1); warp w owns MT 16-row slices of it and every K/V
// fragment it reads from shared memory feeds MT MMAs.  Keys stream through two 64-key
// buffers, one bulk copy per key row (see load_kv_rows_bulk), the next tile requested as
// soon as its buffer is free.  Tiles wholly below the diagonal skip the mask.
template <int DP, int MT>
__global__ void __launch_bounds__(MMA_THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ qo_indptr,
                         const int* __restrict__ seq_lens, const int* __restrict__ block_table,
                         int max_pages, const int* __restrict__ tile_rows,
                         const int* __restrict__ tile_starts, int Hq, int Hkv, int D, int page_size,
                         int num_pages, float scale, int window, int* flag) {
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int STRIDE = Tile<DP>::STRIDE;
    constexpr int CH = Tile<DP>::CHUNKS;
    constexpr int KSTEPS = DP / 16;
    constexpr int DTILES = DP / 8;
    constexpr int ROWS = 64 * MT;  // queries per tile
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + ROWS * STRIDE;                 // 2 buffers
    __nv_bfloat16* sV = sK + 2 * TILE_N * STRIDE;           // 2 buffers
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(sV + 2 * TILE_N * STRIDE);

    // Later tiles of a portion see more keys and run longer: hand them out first (heads
    // vary fastest, so all heads of the longest tile start first) and let the short
    // ones fill the tail of the grid.
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int h = blockIdx.x;
    const int kvh = h / (Hq / Hkv);
    const int row = tile_rows[tile];
    const int q0 = tile_starts[tile];
    const int tok0 = qo_indptr[row];
    const int chunk_len = qo_indptr[row + 1] - tok0;
    const int seq_len = seq_lens[row];
    const int chunk_pos = seq_len - chunk_len;  // absolute position of the portion's first token
    const int* table = block_table + (size_t)row * max_pages;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;      // row within 8
    const int tq = lane & 3;      // column pair

    const int rows_here = min(ROWS, chunk_len - q0);
    const int first_pos = chunk_pos + q0;
    const int last_pos = first_pos + rows_here - 1;
    const int key_end = last_pos + 1;  // causal bound of the tile (<= seq_len)
    const int key_lo = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
    const int first_kt = key_lo / TILE_N;
    const int last_kt = (key_end - 1) / TILE_N;
    const int page_shift = shift_of(page_size);

    // Q tile (rows beyond the portion and columns beyond D are zero)
    for (int c = threadIdx.x; c < ROWS * CH; c += MMA_THREADS) {
        const int r = c / CH;
        const int col = (c % CH) * 8;
        const bool valid = r < rows_here && col < D;
        const __nv_bfloat16* src = valid ? q + (size_t)(tok0 + q0 + r) * q_stride + (size_t)h * D + col : q;
        cp_async16(sQ + r * STRIDE + col, src, valid);
    }
    cp_async_commit();
    if (threadIdx.x == 0) {
        mbar_init(full_bar, 1);
        mbar_init(full_bar + 1, 1);
        fence_barrier_init();
    }
    if (D < DP) {  // columns the copies never write must not hold NaN bit patterns
        for (int idx = threadIdx.x; idx < 4 * TILE_N * (DP - D); idx += MMA_THREADS) {
            const int r = idx / (DP - D);
            sK[r * STRIDE + D + idx % (DP - D)] = __float2bfloat16_rn(0.0f);  // sK and sV are one run of rows
        }
    }
    fence_proxy_async();
    __syncthreads();
#pragma unroll
    for (int ahead = 0; ahead < 2; ++ahead) {
        if (first_kt + ahead <= last_kt)
            load_kv_rows_bulk<DP>(sK + ahead * TILE_N * STRIDE, sV + ahead * TILE_N * STRIDE, k_cache, v_cache, table, max_pages,
                                  num_pages, page_size, page_shift, Hkv, kvh, D, (first_kt + ahead) * TILE_N, key_lo, key_end,
                                  full_bar + ahead);
    }

    float o[MT][DTILES][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < DTILES; ++i) { o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.0f; }
    float m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        m_run[mt][0] = m_run[mt][1] = -INFINITY;
        l_run[mt][0] = l_run[mt][1] = 0.0f;
    }
    const float sl2 = scale * LOG2E;
    const int warp_row0 = warp * 16 * MT;              // first tile row of this warp
    const int warp_pos0 = first_pos + warp_row0;       // its absolute position

    int stage = 0;
    bool timed_out = false;
    for (int kt = first_kt; kt <= last_kt; ++kt) {
        const int use = (kt - first_kt) >> 1;
        const bool landed = mbar_wait(full_bar + stage, use & 1);
        if (kt == first_kt) cp_async_wait<0>();  // the queries
        if (__syncthreads_or(!landed)) {
            timed_out = true;
            break;
        }
        const __nv_bfloat16* tK = sK + stage * TILE_N * STRIDE;
        const __nv_bfloat16* tV = sV + stage * TILE_N * STRIDE;

        // S = Q K^T: this warp's 16*MT queries against the tile's 64 keys
        float s[MT][TILE_N / 8][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < TILE_N / 8; ++nt) { s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a[MT][4];
            const int m = lane >> 3;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int r = warp_row0 + mt * 16 + (m & 1) * 8 + (lane & 7);
                ldmatrix_x4(a[mt], sQ + r * STRIDE + ks * 16 + (m >> 1) * 8);
            }
#pragma unroll
            for (int np = 0; np < TILE_N / 16; ++np) {
                uint32_t b[4];
                const int key = np * 16 + (m >> 1) * 8 + (lane & 7);
                ldmatrix_x4(b, tK + key * STRIDE + ks * 16 + (m & 1) * 8);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_16816(s[mt][2 * np], a[mt], b[0], b[1]);
                    mma_16816(s[mt][2 * np + 1], a[mt], b[2], b[3]);
                }
            }
        }
        // scale, mask (only where the tile reaches the diagonal or the window's edge), online softmax
        const int key_base = kt * TILE_N + tq * 2;
        const bool need_mask = (kt * TILE_N + TILE_N - 1 > warp_pos0) || (window > 0 && kt * TILE_N < warp_pos0 + 16 * MT - window + 1);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int qpos0 = warp_pos0 + mt * 16 + g;
            const int qpos1 = qpos0 + 8;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < TILE_N / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    bool ok0 = true, ok1 = true;
                    if (need_mask) {
                        const int key = key_base + nt * 8 + e;
                        ok0 = key <= qpos0 && (window <= 0 || key > qpos0 - window);
                        ok1 = key <= qpos1 && (window <= 0 || key > qpos1 - window);
                    }
                    s[mt][nt][e] = ok0 ? s[mt][nt][e] * sl2 : -INFINITY;
                    s[mt][nt][2 + e] = ok1 ? s[mt][nt][2 + e] * sl2 : -INFINITY;
                    mx0 = fmaxf(mx0, s[mt][nt][e]);
                    mx1 = fmaxf(mx1, s[mt][nt][2 + e]);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m_run[mt][0], mx0);
            const float mn1 = fmaxf(m_run[mt][1], mx1);
            const float base0 = mn0 == -INFINITY ? 0.0f : mn0;  // a fully masked row stays at zero
            const float base1 = mn1 == -INFINITY ? 0.0f : mn1;
            const float alpha0 = exp2f(m_run[mt][0] - base0);
            const float alpha1 = exp2f(m_run[mt][1] - base1);
            m_run[mt][0] = mn0;
            m_run[mt][1] = mn1;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int nt = 0; nt < TILE_N / 8; ++nt) {
                s[mt][nt][0] = exp2f(s[mt][nt][0] - base0);
                s[mt][nt][1] = exp2f(s[mt][nt][1] - base0);
                s[mt][nt][2] = exp2f(s[mt][nt][2] - base1);
                s[mt][nt][3] = exp2f(s[mt][nt][3] - base1);
                sum0 += s[mt][nt][0] + s[mt][nt][1];
                sum1 += s[mt][nt][2] + s[mt][nt][3];
            }
            l_run[mt][0] = l_run[mt][0] * alpha0 + sum0;
            l_run[mt][1] = l_run[mt][1] * alpha1 + sum1;
#pragma unroll
            for (int dt = 0; dt < DTILES; ++dt) {
                o[mt][dt][0] *= alpha0;
                o[mt][dt][1] *= alpha0;
                o[mt][dt][2] *= alpha1;
                o[mt][dt][3] *= alpha1;
            }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < TILE_N / 16; ++kk) {
            uint32_t a[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
                a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
                a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
                a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
            }
#pragma unroll
            for (int dp = 0; dp < DTILES / 2; ++dp) {
                uint32_t b[4];
                const int m = lane >> 3;
                const int key = kk * 16 + (m & 1) * 8 + (lane & 7);
                ldmatrix_x4_trans(b, tV + key * STRIDE + dp * 16 + (m >> 1) * 8);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_16816(o[mt][2 * dp], a[mt], b[0], b[1]);
                    mma_16816(o[mt][2 * dp + 1], a[mt], b[2], b[3]);
                }
            }
        }
        if (kt + 2 <= last_kt) {  // this buffer's next tile, once every warp is done with it
            __syncthreads();
            load_kv_rows_bulk<DP>(sK + stage * TILE_N * STRIDE, sV + stage * TILE_N * STRIDE, k_cache, v_cache, table, max_pages,
                                  num_pages, page_size, page_shift, Hkv, kvh, D, (kt + 2) * TILE_N, key_lo, key_end,
                                  full_bar + stage);
        }
        stage ^= 1;
    }
    if (timed_out) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_TIMEOUT);
        cp_async_wait<0>();
        for (int st = 0; st < 2; ++st) {
            mbar_wait(full_bar + st, 0, 1u << 10);
            mbar_wait(full_bar + st, 1, 1u << 10);
        }
        return;
    }

    // finish: row sums across the quad, normalise, store
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float l0 = l_run[mt][0], l1 = l_run[mt][1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f;
        const float inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
        const int r0 = warp_row0 + mt * 16 + g;
        const int r1 = r0 + 8;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            const int col = dt * 8 + tq * 2;
            if (col < D) {
                if (r0 < rows_here) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[mt][dt][0] * inv0, o[mt][dt][1] * inv0);
                    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + q0 + r0) * out_stride + (size_t)h * D + col) = v;
                }
                if (r1 < rows_here) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[mt][dt][2] * inv1, o[mt][dt][3] * inv1);
                    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + q0 + r1) * out_stride + (size_t)h * D + col) = v;
                }
            }
        }
    }
}

// ------------------------------------------------------------------ decode: split-KV
// grid (rows, Hkv, splits).  The G = Hq/Hkv query heads of one KV head are the
// 16-row M tile (rows >= G are zero).  Split s covers absolute keys
// [s*DEC_SPLIT, (s+1)*DEC_SPLIT); warp w takes keys w*16..w*16+15 of every
// 64-key tile.  Partials (unnormalised O, running max, running sum) go to
// scratch; the merge kernel combines splits in order.
template <int DP>
__global__ void __launch_bounds__(MMA_THREADS)
attention_decode_split_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                              const __nv_bfloat16* __restrict__ k_cache,
                              const __nv_bfloat16* __restrict__ v_cache,
                              const int* __restrict__ seq_lens, const int* __restrict__ block_table,
                              int max_pages, const int* __restrict__ decode_rows,
                              const int* __restrict__ decode_tokens, int Hq, int Hkv, int D,
                              int page_size, int num_pages, float scale, int window, int num_splits,
                              float* __restrict__ part_o, float* __restrict__ part_ml, int* flag) {
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int STRIDE = Tile<DP>::STRIDE;
    constexpr int CH = Tile<DP>::CHUNKS;
    constexpr int KSTEPS = DP / 16;
    constexpr int DTILES = DP / 8;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // 16 rows
    __nv_bfloat16* sK = sQ + 16 * STRIDE;                             // DEC_STAGES stages of 64 keys
    __nv_bfloat16* sV = sK + DEC_STAGES * TILE_N * STRIDE;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(sV + DEC_STAGES * TILE_N * STRIDE);  // one per stage

    const int slot = blockIdx.x;
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int row = decode_rows[slot];
    const int token = decode_tokens[slot];
    const int seq_len = seq_lens[row];
    const int G = Hq / Hkv;
    const int qpos = seq_len - 1;
    const int key_lo_all = (window > 0 && qpos + 1 > window) ? qpos + 1 - window : 0;
    const int key0 = max(split * DEC_SPLIT, (key_lo_all / TILE_N) * TILE_N);
    const int key_end = min((split + 1) * DEC_SPLIT, seq_len);
    if (key0 >= key_end || split * DEC_SPLIT + DEC_SPLIT <= key_lo_all) return;  // nothing of this split is visible
    const int* table = block_table + (size_t)row * max_pages;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int tq = lane & 3;

    for (int c = threadIdx.x; c < 16 * CH; c += MMA_THREADS) {
        const int r = c / CH;
        const int col = (c % CH) * 8;
        const bool valid = r < G && col < D;
        const __nv_bfloat16* src = valid ? q + (size_t)token * q_stride + (size_t)(kvh * G + r) * D + col : q;
        cp_async16(sQ + r * STRIDE + col, src, valid);
    }
    cp_async_commit();  // the queries
    const int first_tile = key0 / TILE_N;
    const int last_tile = (key_end - 1) / TILE_N;
    const int page_shift = shift_of(page_size);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int st = 0; st < DEC_STAGES; ++st) mbar_init(full_bar + st, 1);
        fence_barrier_init();
    }
    if (D < DP) {  // columns the copies never write must not hold NaN bit patterns
        for (int idx = threadIdx.x; idx < 2 * DEC_STAGES * TILE_N * (DP - D); idx += MMA_THREADS) {
            const int r = idx / (DP - D);
            const int col = D + idx % (DP - D);
            sK[r * STRIDE + col] = __float2bfloat16_rn(0.0f);  // sK and sV are one contiguous run of rows
        }
    }
    fence_proxy_async();
    __syncthreads();
    // prologue: request the first DEC_STAGES tiles (a whole split when DEC_SPLIT == DEC_STAGES * TILE_N)
#pragma unroll
    for (int ahead = 0; ahead < DEC_STAGES; ++ahead) {
        if (first_tile + ahead <= last_tile)
            load_kv_rows_bulk<DP>(sK + ahead * TILE_N * STRIDE, sV + ahead * TILE_N * STRIDE, k_cache, v_cache, table, max_pages,
                                  num_pages, page_size, page_shift, Hkv, kvh, D, (first_tile + ahead) * TILE_N, key_lo_all,
                                  key_end, full_bar + ahead);
    }

    uint32_t qf[KSTEPS][4];
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};
    const float sl2 = scale * LOG2E;

    int stage = 0;
    bool timed_out = false;
    for (int kt = first_tile; kt <= last_tile; ++kt) {
        const int use = (kt - first_tile) / DEC_STAGES;  // how often this stage has been filled before
        const bool landed = mbar_wait(full_bar + stage, use & 1);
        if (kt == first_tile) cp_async_wait<0>();  // the queries
        if (__syncthreads_or(!landed)) {  // every thread has tile kt (and the queries)
            timed_out = true;
            break;
        }
        if (kt == first_tile) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const int m = lane >> 3;
                const int r = (m & 1) * 8 + (lane & 7);
                const int col = ks * 16 + (m >> 1) * 8;
                ldmatrix_x4(qf[ks], sQ + r * STRIDE + col);
            }
        }
        const __nv_bfloat16* tK = sK + stage * TILE_N * STRIDE + warp * 16 * STRIDE;
        const __nv_bfloat16* tV = sV + stage * TILE_N * STRIDE + warp * 16 * STRIDE;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.0f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t b[4];
            const int m = lane >> 3;
            const int key = (m >> 1) * 8 + (lane & 7);
            const int col = ks * 16 + (m & 1) * 8;
            ldmatrix_x4(b, tK + key * STRIDE + col);
            mma_16816(s[0], qf[ks], b[0], b[1]);
            mma_16816(s[1], qf[ks], b[2], b[3]);
        }
        const int key_base = kt * TILE_N + warp * 16 + tq * 2;
        // every row of the M tile has the same query position
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key_base + nt * 8 + e;
                const bool ok = key < key_end && key >= key_lo_all;
                s[nt][e] = ok ? s[nt][e] * sl2 : -INFINITY;
                s[nt][2 + e] = ok ? s[nt][2 + e] * sl2 : -INFINITY;
            }
        }
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0);
        const float mn1 = fmaxf(m_run[1], mx1);
        const float base0 = mn0 == -INFINITY ? 0.0f : mn0;
        const float base1 = mn1 == -INFINITY ? 0.0f : mn1;
        const float alpha0 = exp2f(m_run[0] - base0);
        const float alpha1 = exp2f(m_run[1] - base1);
        m_run[0] = mn0;
        m_run[1] = mn1;
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - base0);
            s[nt][1] = exp2f(s[nt][1] - base0);
            s[nt][2] = exp2f(s[nt][2] - base1);
            s[nt][3] = exp2f(s[nt][3] - base1);
            sum0 += s[nt][0] + s[nt][1];
            sum1 += s[nt][2] + s[nt][3];
        }
        l_run[0] = l_run[0] * alpha0 + sum0;
        l_run[1] = l_run[1] * alpha1 + sum1;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            o[dt][0] *= alpha0;
            o[dt][1] *= alpha0;
            o[dt][2] *= alpha1;
            o[dt][3] *= alpha1;
        }
        uint32_t a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
            uint32_t b[4];
            const int m = lane >> 3;
            const int key = (m & 1) * 8 + (lane & 7);
            const int col = dp * 16 + (m >> 1) * 8;
            ldmatrix_x4_trans(b, tV + key * STRIDE + col);
            mma_16816(o[2 * dp], a, b[0], b[1]);
            mma_16816(o[2 * dp + 1], a, b[2], b[3]);
        }
        if (kt + DEC_STAGES <= last_tile) {  // more tiles than buffers: refill this one once everyone is done with it
            __syncthreads();
            load_kv_rows_bulk<DP>(sK + stage * TILE_N * STRIDE, sV + stage * TILE_N * STRIDE, k_cache, v_cache, table, max_pages,
                                  num_pages, page_size, page_shift, Hkv, kvh, D, (kt + DEC_STAGES) * TILE_N, key_lo_all, key_end,
                                  full_bar + stage);
        }
        stage = (stage + 1) % DEC_STAGES;
    }
    if (timed_out) {
        // A copy did not land in time.  Say so, give the copies still in flight one more
        // bounded wait (they target this block's shared memory), and leave without a result.
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_TIMEOUT);
        cp_async_wait<0>();
        for (int st = 0; st < DEC_STAGES; ++st) {
            mbar_wait(full_bar + st, 0, 1u << 10);
            mbar_wait(full_bar + st, 1, 1u << 10);
        }
        return;
    }
    __syncthreads();  // every warp is done with the tiles before they become the merge buffer

    // combine the four warps (in warp order) through shared memory
    float l0 = l_run[0], l1 = l_run[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    constexpr int OSTRIDE = DP + 8;                   // fp32 row stride of the merge buffer
    float* sO = reinterpret_cast<float*>(smem_raw);   // [4 warps][16 rows][OSTRIDE]
    float* sM = sO + 4 * 16 * OSTRIDE;                // [4][16]
    float* sL = sM + 4 * 16;                          // [4][16]
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
        const int col = dt * 8 + tq * 2;
        float* base = sO + (size_t)warp * 16 * OSTRIDE;
        *reinterpret_cast<float2*>(base + g * OSTRIDE + col) = make_float2(o[dt][0], o[dt][1]);
        *reinterpret_cast<float2*>(base + (g + 8) * OSTRIDE + col) = make_float2(o[dt][2], o[dt][3]);
    }
    if (tq == 0) {
        sM[warp * 16 + g] = m_run[0];
        sM[warp * 16 + g + 8] = m_run[1];
        sL[warp * 16 + g] = l0;
        sL[warp * 16 + g + 8] = l1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += MMA_THREADS) {
        const int r = idx / D;
        const int d = idx % D;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) big = fmaxf(big, sM[w * 16 + r]);
        float acc = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sM[w * 16 + r];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - big);
            acc += sO[((size_t)w * 16 + r) * OSTRIDE + d] * f;
            den += sL[w * 16 + r] * f;
        }
        const size_t pidx = ((size_t)slot * Hq + (kvh * G + r)) * num_splits + split;
        part_o[pidx * D + d] = acc;
        if (d == 0) {
            part_ml[pidx * 2] = big;
            part_ml[pidx * 2 + 1] = den;
        }
    }
}

// grid (rows, Hq); combines the splits a row has, in split order.
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o,
                                              const float* __restrict__ part_ml,
                                              const int* __restrict__ seq_lens,
                                              const int* __restrict__ decode_rows,
                                              const int* __restrict__ decode_tokens,
                                              __nv_bfloat16* __restrict__ out, int out_stride, int Hq,
                                              int D, int window, int num_splits) {
    pdl_wait();
    const int slot = blockIdx.x;
    const int h = blockIdx.y;
    const int row = decode_rows[slot];
    const int token = decode_tokens[slot];
    const int seq_len = seq_lens[row];
    const int qpos = seq_len - 1;
    const int key_lo = (window > 0 && qpos + 1 > window) ? qpos + 1 - window : 0;
    const int first = key_lo / DEC_SPLIT;
    const int last = min((seq_len - 1) / DEC_SPLIT, num_splits - 1);
    const size_t base = ((size_t)slot * Hq + h) * num_splits;
    float big = -INFINITY;
    for (int s = first; s <= last; ++s) big = fmaxf(big, part_ml[(base + s) * 2]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f, den = 0.0f;
        for (int s = first; s <= last; ++s) {
            const float ms = part_ml[(base + s) * 2];
            const float f = ms == -INFINITY ? 0.0f : exp2f(ms - big);
            acc += part_o[(base + s) * D + d] * f;
            den += part_ml[(base + s) * 2 + 1] * f;
        }
        out[(size_t)token * out_stride + (size_t)h * D + d] = __float2bfloat16_rn(den > 0.0f ? acc / den : 0.0f);
    }
}

// ------------------------------------------------------------------ host-side launchers
template <int DP, int MT>
static size_t prefill_smem() {
    return (size_t)(64 * MT + 4 * TILE_N) * Tile<DP>::STRIDE * sizeof(__nv_bfloat16) + 2 * sizeof(uint64_t);
}

template <int DP>
static size_t decode_smem() {
    const size_t tiles = (size_t)(16 + 2 * DEC_STAGES * TILE_N) * Tile<DP>::STRIDE * sizeof(__nv_bfloat16) + DEC_STAGES * sizeof(uint64_t);
    const size_t merge = (size_t)(4 * 16 * (DP + 8) + 2 * 4 * 16) * sizeof(float);
    return tiles > merge ? tiles : merge;
}

static int padded_dim(int D) {
    if (D % 16 != 0 || D < 16 || D > 256) return 0;
    if (D <= 32) return 32;
    if (D <= 64) return 64;
    if (D <= 128) return 128;
    return 256;
}

// Queries per tile of the prefill kernel for a head size: 128 up to a padded size of 128, else 64.
static inline int prefill_tile_rows(int D) { return padded_dim(D) <= 128 ? 128 : 64; }

template <int DP, int MT>
static int launch_prefill(const __nv_bfloat16* q, int q_stride, __nv_bfloat16* out, int out_stride,
                          const __nv_bfloat16* k_cache, const __nv_bfloat16* v_cache,
                          const int* qo_indptr, const int* seq_lens, const int* block_table,
                          int max_pages, const int* tile_rows, const int* tile_starts, int num_tiles,
                          int Hq, int Hkv, int D, int page_size, int num_pages, float scale,
                          int window, int* flag, cudaStream_t stream) {
    const size_t smem = prefill_smem<DP, MT>();
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DP, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(Hq, num_tiles);
    kb_launch(attention_prefill_kernel<DP, MT>, dim3(grid), dim3(MMA_THREADS), smem, stream, 
        q, q_stride, out, out_stride, k_cache, v_cache, qo_indptr, seq_lens, block_table, max_pages,
        tile_rows, tile_starts, Hq, Hkv, D, page_size, num_pages, scale, window, flag);
    return kb_launch_result();
}

template <int DP>
static int launch_decode(const __nv_bfloat16* q, int q_stride, const __nv_bfloat16* k_cache,
                         const __nv_bfloat16* v_cache, const int* seq_lens, const int* block_table,
                         int max_pages, const int* decode_rows, const int* decode_tokens, int num_rows,
                         int Hq, int Hkv, int D, int page_size, int num_pages, float scale, int window,
                         int num_splits, float* part_o, float* part_ml, int* flag, cudaStream_t stream) {
    const size_t smem = decode_smem<DP>();
    cudaError_t e = cudaFuncSetAttribute(attention_decode_split_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(num_rows, Hkv, num_splits);
    kb_launch(attention_decode_split_kernel<DP>, dim3(grid), dim3(MMA_THREADS), smem, stream, 
        q, q_stride, k_cache, v_cache, seq_lens, block_table, max_pages, decode_rows, decode_tokens,
        Hq, Hkv, D, page_size, num_pages, scale, window, num_splits, part_o, part_ml, flag);
    return kb_launch_result();
}

