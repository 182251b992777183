// Weight-streaming matrix product for a few tokens (decode):
//     out[M, N] = x[M, K] . W[N, K]^T (+ bias),   M <= 16, bf16 in, fp32 accumulate,
// optionally with the SiLU gate fused in:  out[M, N/2] = silu(x.Wg^T) * (x.Wu^T)
// where Wg = W[:N/2] and Wu = W[N/2:] (kairyu/models/layers.py:244).
//
// At these M the product is bound by reading W once from HBM.  The weights are the
// 16-row operand of mma.sync m16n8k16 and the tokens its 8 columns, so W is
// consumed at tensor-core rate straight from registers: every thread loads 32
// contiguous bytes of a weight row and 32 of a token row; because a dot product
// does not care in which order k is summed, those 16 values are handed to four
// MMAs as their (k, k+8) pairs without any shuffle.  A block owns 16 weight rows; its
// warps split K and their partial sums are added in warp order through shared
// memory, so the result does not depend on timing.
//
// RMSNorm around the product, without a kernel of its own (kairyu/models/layers.py:21-46 is the
// norm, kairyu/models/llama.py:88-101 the residual arrangement).  With y = rmsnorm(r) * g feeding
// a product, (y . W^T)[m] = rstd[m] * ((r[m] * g) . W^T): the product before can leave r * g
// (rounded to bf16) and the sum of r^2, and this product scales its rows by rstd in the epilogue.
//   * fold:  the epilogue adds the result to the fp32 residual r (in place), writes bf16(r * g)
//     for the next product and, per block, the partial sums of r^2 over the block's columns;
//   * scale: the epilogue multiplies row m by rsqrt(sum of the partial sums / H + eps) before
//     bias and gate.  The partial sums are added in block order, so the result does not depend
//     on timing.
#include "common.cuh"

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define SK_UNROLL 2
#define SK_STEP 64  // k per step: four lanes of a weight row load 32 bytes each, one full 128-byte line
#define SK_SUM_BLOCKS 384  // a scaling epilogue adds up to this many partial sums per row

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Reg8 {
    uint32_t r[8];
};

// What the epilogue does beside the product (all pointers null: nothing).
struct SkinnyFusion {
    // scale: rows come unnormalised; in_sumsq[b * 16 + m] are the producer's partial sums of row m
    const float* in_sumsq;
    int in_blocks;
    float in_inv_hidden;
    float in_eps;
    // fold: residual[m, n] += result; values[m, n] = bf16(residual * norm_w[n]); out_sumsq[block * 16 + m]
    float* residual;
    int ldr;
    const void* norm_w;
    int norm_w_bf16;
    __nv_bfloat16* values;
    int ldv;
    float* out_sumsq;
    // rope: the product is q | k | v of attention (heads of D columns: Hq, then Hkv, then Hkv).  The
    // epilogue rotates q and k by the token's position (rotate-half over the whole head,
    // kairyu/models/layers.py:129-148), writes q to out and k and v into their cache pages
    // (kairyu/engine/core/kv_pool.py:171-348).  A block then owns columns j..j+7 and D/2+j..D/2+j+7
    // of one head, so that both elements of a rotated pair meet in one warp.
    const float* rope_cos;  // [max_pos, D/2] fp32; null: no rope work
    const float* rope_sin;
    int rope_max_pos;
    int Hq, Hkv, D;
    const int* positions;    // [M]
    const int* row_ids;      // [M]
    const int* block_table;  // [rows, max_pages]
    int max_pages;
    const int* write_from;   // [rows]
    __nv_bfloat16* k_cache;  // [num_pages, page_size, Hkv, D]
    __nv_bfloat16* v_cache;
    int page_size, num_pages;
    int* flag;
};

// streaming 32-byte load of weights (sm_100 has 256-bit loads): read once, keep out of L1
__device__ __forceinline__ Reg8 load_stream32(const void* p) {
    Reg8 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
                 : "l"(p));
    return v;
}
// 32-byte load of activations: small, shared by every block, kept in L1
__device__ __forceinline__ Reg8 load_cached32(const void* p) {
    Reg8 v;
    asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
                 : "l"(p));
    return v;
}

// NT: token tiles of 8 (1 or 2).  GATED: warps 0..3 walk the gate rows and warps
// 4..7 the rows N/2 further down (the "up" half); the epilogue writes silu(gate) * up.
// MINB: blocks the compiler keeps room for on an SM (2 or 3).  A grid that does not fit at two
// blocks per SM (q/k/v: 384 blocks, the head: thousands) runs faster at three, with 80
// registers a thread and a few spilled bytes; one that fits (o, down: 256 blocks) does not.
// FUSED: the epilogue does norm work (SkinnyFusion); the plain instantiation carries none of it.
template <int NT, bool GATED, typename TO, int MINB, bool FUSED>
__global__ void __launch_bounds__(SK_THREADS, MINB)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                   int ldw, const __nv_bfloat16* __restrict__ bias, TO* __restrict__ out, int ldo,
                   int M, int N, int K, int rows_per_block_arg, SkinnyFusion fusion) {
    // Only the two-per-SM variant takes a runtime row count: at three per SM (80 registers) the
    // extra predicates spill into the main loop.
    const int rows_per_block = MINB == 2 ? rows_per_block_arg : 16;
    pdl_trigger();
    constexpr int HALVES = GATED ? 2 : 1;
    constexpr int KWARPS = SK_WARPS / HALVES;  // warps that split K for one half
    __shared__ float partial[SK_WARPS][NT][16][8 + 1];
    constexpr int SUM_TOKENS = NT * 8;                 // token rows the epilogue may scale
    constexpr int SUM_CHUNKS = SK_THREADS / SUM_TOKENS;  // threads (chunks of blocks) that share a token's partial sums
    constexpr int SUM_ROUNDS = SK_SUM_BLOCKS / SUM_CHUNKS;
    __shared__ float sums[SUM_CHUNKS][SUM_TOKENS + 1];  // [chunk of blocks][token] partial sums of the rows' squares
    __shared__ float row_scale[16];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int tq = lane & 3;
    const int half = warp / KWARPS;
    const int kwarp = warp % KWARPS;
    const int rows_out = GATED ? N / 2 : N;      // output columns
    // A block owns rows_per_block (<= 16) weight rows: fewer than 16 leaves rows of the MMA tile
    // idle, which costs nothing here, and lets the host pick a grid that fills every SM evenly.
    const int n0 = blockIdx.x * rows_per_block;  // first weight row (and output column) of the block
    // Weight row (= output column) of the block's local row r.  With rope work the 16 rows are two
    // runs of 8, half a head apart.
    const bool roped = FUSED && fusion.rope_cos != nullptr;
    const int rope_half = roped ? fusion.D >> 1 : 0;
    int rope_base = 0;
    if (roped) {
        const int per_head = rope_half >= 8 ? rope_half >> 3 : 1;  // blocks a head (the host refuses heads under 16)
        rope_base = (blockIdx.x / per_head) * fusion.D + (blockIdx.x % per_head) * 8;
    }
    auto column_of = [&](int r) { return roped ? rope_base + (r & 7) + ((r & 8) ? rope_half : 0) : n0 + r; };

    // K is cut into SK_STEP-wide steps; warp kwarp takes steps kwarp, kwarp + KWARPS, ...
    const int steps = (K + SK_STEP - 1) / SK_STEP;
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;

    const int row_lo = column_of(g);
    const int row_hi = column_of(g + 8);
    const bool lo_ok = g < rows_per_block && row_lo < rows_out;
    const bool hi_ok = g + 8 < rows_per_block && row_hi < rows_out;
    const __nv_bfloat16* w_lo = w + (size_t)(half * rows_out + (lo_ok ? row_lo : 0)) * ldw;
    const __nv_bfloat16* w_hi = w + (size_t)(half * rows_out + (hi_ok ? row_hi : 0)) * ldw;
    const __nv_bfloat16* x_row[NT];
    bool x_ok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        x_ok[t] = t * 8 + g < M;
        x_row[t] = x + (size_t)(x_ok[t] ? t * 8 + g : 0) * ldx;
    }
    Reg8 zero;
#pragma unroll
    for (int i = 0; i < 8; ++i) zero.r[i] = 0u;

    // Two register sets: the loads of the next SK_UNROLL steps are issued before the
    // MMAs of the current ones, so a warp always has a batch in flight.
    Reg8 a_lo[2][SK_UNROLL], a_hi[2][SK_UNROLL], b[2][SK_UNROLL][NT];
    auto load_weights = [&](int set, int step0) {
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int k = (step0 + u * KWARPS) * SK_STEP + tq * 16;
            const bool k_ok = k < K;  // K % 16 == 0, so a 32-byte load is all in or all out
            a_lo[set][u] = (k_ok && lo_ok) ? load_stream32(w_lo + k) : zero;
            a_hi[set][u] = (k_ok && hi_ok) ? load_stream32(w_hi + k) : zero;
        }
    };
    auto load_tokens = [&](int set, int step0) {
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int k = (step0 + u * KWARPS) * SK_STEP + tq * 16;
            const bool k_ok = k < K;
#pragma unroll
            for (int t = 0; t < NT; ++t) b[set][u][t] = (k_ok && x_ok[t]) ? load_cached32(x_row[t] + k) : zero;
        }
    };
    auto load_batch = [&](int set, int step0) {
        load_weights(set, step0);
        load_tokens(set, step0);
    };
    // The 16 values a thread holds of a row feed four MMAs: MMA j takes values 4j..4j+3
    // as its (k, k+1) and (k+8, k+9) pairs.  Which k a value is called does not matter to
    // a dot product as long as the weight and the token agree, and they do: both come
    // from the same 32 bytes of their rows.
    auto mma_batch = [&](int set) {
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    mma_bf16(acc[t], a_lo[set][u].r[2 * j], a_hi[set][u].r[2 * j], a_lo[set][u].r[2 * j + 1],
                             a_hi[set][u].r[2 * j + 1], b[set][u][t].r[2 * j], b[set][u][t].r[2 * j + 1]);
    };
    constexpr int STRIDE = KWARPS * SK_UNROLL;
    int step0 = kwarp;
    // The weights do not depend on the kernel before this one: their first loads go out
    // before the wait, the tokens (that kernel's output) after it.
    load_weights(0, step0);
    // rope: what this thread's (token, row) needs of the token's position, used in the epilogue: cos and
    // sin for q and k, the slot in the cache for k and v.  Positions, row ids and block tables are
    // written by the step's copy from the host and the tables never change, so these dependent loads
    // need not wait for the kernel before this one: they run while the first weights are on their way.
    // (kept in shared memory, each thread its own words: registers are short in the main loop)
    __shared__ float rope_c[FUSED ? NT * 8 * 16 : 1], rope_s[FUSED ? NT * 8 * 16 : 1];
    __shared__ long long rope_slot[FUSED ? NT * 8 * 16 : 1];
    if (roped && threadIdx.x < NT * 8 * 16) {
        float held_cos = 1.0f, held_sin = 0.0f;
        long long held_slot = -1;
        const int r = threadIdx.x & 15;
        const int token = threadIdx.x >> 4;
        if (token < M) {
            const int column = column_of(r);
            const int head = column / fusion.D;
            const int pos = fusion.positions[token];
            if (pos < 0 || pos >= fusion.rope_max_pos) {
                if (fusion.flag) atomicOr(fusion.flag, KB_FLAG_BAD_POS);  // left unrotated and unwritten
            } else {
                if (head < fusion.Hq + fusion.Hkv) {
                    const int i = column - head * fusion.D - ((r & 8) ? rope_half : 0);
                    held_cos = fusion.rope_cos[(size_t)pos * rope_half + i];
                    held_sin = fusion.rope_sin[(size_t)pos * rope_half + i];
                }
                if (head >= fusion.Hq && fusion.k_cache != nullptr) {
                    const int row = fusion.row_ids[token];
                    if (pos >= fusion.write_from[row]) {
                        const int page_index = pos / fusion.page_size;
                        const int page = page_index < fusion.max_pages ? fusion.block_table[(size_t)row * fusion.max_pages + page_index] : -1;
                        if (page < 0 || page >= fusion.num_pages) {
                            if (fusion.flag) atomicOr(fusion.flag, KB_FLAG_BAD_PAGE);
                        } else {
                            held_slot = (long long)page * fusion.page_size + (pos - page_index * fusion.page_size);
                        }
                    }
                }
            }
        }
        rope_c[threadIdx.x] = held_cos;
        rope_s[threadIdx.x] = held_sin;
        rope_slot[threadIdx.x] = held_slot;
    }
    pdl_wait();
    load_tokens(0, step0);
    // scale: thread (chunk, token) adds every 16th block's partial sum of its token's row; the
    // loads overlap the first weights' way from memory
    float my_sum = 0.0f;
    if (FUSED && fusion.in_sumsq != nullptr) {
        // up to SK_SUM_BLOCKS blocks; the loads go out together, not one per round trip
        float part[SUM_ROUNDS];
#pragma unroll
        for (int i = 0; i < SUM_ROUNDS; ++i) {
            const int b = threadIdx.x / SUM_TOKENS + SUM_CHUNKS * i;
            part[i] = b < fusion.in_blocks ? fusion.in_sumsq[b * 16 + threadIdx.x % SUM_TOKENS] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < SUM_ROUNDS; ++i) my_sum += part[i];
    }
    // fold: this thread's element of the residual and of the norm weight, asked for now and used in the epilogue
    float held_residual = 0.0f, held_weight = 0.0f;
    if (FUSED && fusion.residual != nullptr && threadIdx.x < NT * 8 * 16) {
        const int r = threadIdx.x & 15;
        const int token = threadIdx.x >> 4;
        const int n = column_of(r);
        if (token < M && r < rows_per_block && n < rows_out) {
            held_residual = fusion.residual[(size_t)token * fusion.ldr + n];
            held_weight = fusion.norm_w_bf16 ? __bfloat162float(((const __nv_bfloat16*)fusion.norm_w)[n]) : ((const float*)fusion.norm_w)[n];
        }
    }
    while (true) {
        load_batch(1, step0 + STRIDE);  // past the end: all zero, no memory touched
        mma_batch(0);
        step0 += STRIDE;
        if (step0 >= steps) break;
        load_batch(0, step0 + STRIDE);
        mma_batch(1);
        step0 += STRIDE;
        if (step0 >= steps) break;
    }

    // acc[t]: c0,c1 = (row g, tokens t*8 + 2tq, +1); c2,c3 = (row g+8, same tokens)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        partial[warp][t][g][2 * tq] = acc[t][0];
        partial[warp][t][g][2 * tq + 1] = acc[t][1];
        partial[warp][t][g + 8][2 * tq] = acc[t][2];
        partial[warp][t][g + 8][2 * tq + 1] = acc[t][3];
    }
    if (FUSED) sums[threadIdx.x / SUM_TOKENS][threadIdx.x % SUM_TOKENS] = my_sum;
    __syncthreads();
    if (FUSED && fusion.in_sumsq != nullptr) {
        if (threadIdx.x < SUM_TOKENS) {
            float total = 0.0f;
#pragma unroll
            for (int c = 0; c < SUM_CHUNKS; ++c) total += sums[c][threadIdx.x];
            row_scale[threadIdx.x] = rsqrtf(total * fusion.in_inv_hidden + fusion.in_eps);
        }
        __syncthreads();
    }
    // one thread per (token, row): rows fastest so that stores of a token are contiguous.  Whole
    // warps are inside the loop or outside it (its bound is a multiple of 32).
    for (int idx = threadIdx.x; idx < NT * 8 * 16; idx += SK_THREADS) {
        const int r = idx & 15;
        const int token = idx >> 4;
        const int t = token >> 3;
        const int col = token & 7;
        const int n = column_of(r);
        const bool valid = token < M && r < rows_per_block && n < rows_out;
        float result = 0.0f;
        if (valid) {
            float value[HALVES];
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                float sum = 0.0f;
#pragma unroll
                for (int wp = 0; wp < KWARPS; ++wp) sum += partial[h * KWARPS + wp][t][r][col];
                if (FUSED && fusion.in_sumsq != nullptr) sum *= row_scale[token];
                if (bias) sum += __bfloat162float(bias[h * rows_out + n]);
                value[h] = sum;
            }
            result = value[0];
            if (GATED) result = value[0] / (1.0f + expf(-value[0])) * value[HALVES - 1];
        }
        if (roped) {
            // the other element of the rotated pair is eight rows on, in the same warp;
            // rotate_half(u) = cat(-u[half:], u[:half])
            const float partner = __shfl_xor_sync(0xffffffffu, result, 8);
            const float held_cos = rope_c[idx], held_sin = rope_s[idx];  // idx == threadIdx.x: the loop runs once
            const long long held_slot = rope_slot[idx];
            const int head = n / fusion.D;
            float rotated = result;
            if (head < fusion.Hq + fusion.Hkv)
                rotated = (r & 8) ? result * held_cos + partner * held_sin : result * held_cos - partner * held_sin;
            if (valid) {
                const __nv_bfloat16 rounded = __float2bfloat16_rn(rotated);
                if (head < fusion.Hq) {
                    reinterpret_cast<__nv_bfloat16*>(out)[(size_t)token * ldo + n] = rounded;
                } else if (held_slot >= 0) {
                    const bool is_k = head < fusion.Hq + fusion.Hkv;
                    const int kvh = head - fusion.Hq - (is_k ? 0 : fusion.Hkv);
                    __nv_bfloat16* cache = is_k ? fusion.k_cache : fusion.v_cache;
                    cache[((size_t)held_slot * fusion.Hkv + kvh) * fusion.D + (n - head * fusion.D)] = rounded;
                }
            }
            continue;
        }
        if (!FUSED || fusion.residual == nullptr) {
            if (valid) out[(size_t)token * ldo + n] = from_float<TO>(result);
            continue;
        }
        float square = 0.0f;
        if (valid) {
            // (NT * 8 * 16 <= SK_THREADS: the loop runs once and idx == threadIdx.x, as when the values were fetched)
            const float sum = held_residual + result;
            fusion.residual[(size_t)token * fusion.ldr + n] = sum;
            fusion.values[(size_t)token * fusion.ldv + n] = __float2bfloat16_rn(sum * held_weight);
            square = sum * sum;
        }
        // the 16 rows of a token sit in 16 neighbouring lanes
        square += __shfl_xor_sync(0xffffffffu, square, 8);
        square += __shfl_xor_sync(0xffffffffu, square, 4);
        square += __shfl_xor_sync(0xffffffffu, square, 2);
        square += __shfl_xor_sync(0xffffffffu, square, 1);
        if (r == 0) fusion.out_sumsq[(size_t)blockIdx.x * 16 + token] = square;
    }
}

// rows per block and whether three blocks go on an SM, for (rows of output, token tiles, gated)
static void skinny_grid(int rows_out, bool single_tile_plain, bool gated, int& rows_per_block, bool& three) {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 148;
    }
    // Grid: one wave that fills every SM evenly where the rows allow it (rows per block between
    // 8 and 16, two blocks per SM); else 16-row blocks, three to an SM, for the plain single-tile
    // product; the others (gated, two token tiles) run two blocks per SM, the gated one with the
    // rows per block that fill its last wave best.
    rows_per_block = 16;
    three = false;
    if (single_tile_plain) {
        const int fit2 = (rows_out + 2 * sms - 1) / (2 * sms);
        if (fit2 <= 16)
            rows_per_block = fit2 < 8 ? 8 : fit2;
        else
            three = true;
    } else if (gated && rows_out > 2 * sms * 16) {
        // Several waves of two blocks per SM: the last wave should be nearly full.  Cost of a
        // choice = whole waves x rows per block (a wave's time goes with the rows its blocks
        // stream); between 12 and 16 rows the fixed cost of a block does not change the order.
        // (Llama-3.1-8B gate/up, 14,336 rows: 13 rows, 3.73 waves; measured 0.8 % of the decode
        // step faster than 16 rows and 3.03 waves.)
        long best = -1;
        for (int rows = 16; rows >= 12; --rows) {
            const long blocks = (rows_out + rows - 1) / rows;
            const long waves = (blocks + 2 * sms - 1) / (2 * sms);
            if (best < 0 || waves * rows < best) {
                best = waves * rows;
                rows_per_block = rows;
            }
        }
    }
}

template <int NT, bool GATED>
static int launch_skinny(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* w, int ldw,
                         const __nv_bfloat16* bias, void* out, int out_fp32, int ldo, int M, int N, int K,
                         const SkinnyFusion& fusion, cudaStream_t stream) {
    const int rows_out = GATED ? N / 2 : N;
    int rows_per_block;
    bool three;
    skinny_grid(rows_out, !GATED && NT == 1, GATED, rows_per_block, three);
    if (fusion.rope_cos != nullptr) rows_per_block = 16;  // two runs of eight columns, half a head apart
    const int blocks = (rows_out + rows_per_block - 1) / rows_per_block;
    const bool fused = fusion.in_sumsq != nullptr || fusion.residual != nullptr || fusion.rope_cos != nullptr;
#define GO(TO_, MINB_, F_) kb_launch(gemm_skinny_kernel<NT, GATED, TO_, MINB_, F_>, dim3(blocks), dim3(SK_THREADS), 0, stream, x, ldx, w, ldw, bias, (TO_*)out, ldo, M, N, K, rows_per_block, fusion)
#define PICK(TO_) do { if (three) { if (fused) GO(TO_, 3, true); else GO(TO_, 3, false); } else { if (fused) GO(TO_, 2, true); else GO(TO_, 2, false); } } while (0)
    if (out_fp32) PICK(float); else PICK(__nv_bfloat16);
#undef PICK
#undef GO
    return kb_launch_result();
}

// x: [M, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), bias: [N] bf16 or null,
// out: [M, N] (or [M, N/2] when gated) bf16 or fp32.  Needs M <= 16, K % 16 == 0 and
// 32-byte aligned rows; anything else is refused (the caller has the library product).
static int skinny_entry(const void* x, int ldx, const void* w, int ldw, const void* bias, void* out, int out_fp32, int ldo,
                        int M, int N, int K, int gated, const SkinnyFusion& fusion, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (!x || !w || (!out && !fusion.residual)) return KB_ERR_NULL;
    if (M < 1 || M > 16 || K < 16 || K % 16 != 0 || ldx % 16 != 0 || ldw % 16 != 0) return KB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)x | (uintptr_t)w) % 32 != 0) return KB_ERR_UNSUPPORTED_SIZE;
    if (gated && N % 2 != 0) return KB_ERR_BAD_ARG;
    if (fusion.residual && (gated || !fusion.norm_w || !fusion.values || !fusion.out_sumsq)) return KB_ERR_BAD_ARG;
    if (fusion.in_sumsq && (fusion.in_blocks < 1 || fusion.in_blocks > SK_SUM_BLOCKS)) return KB_ERR_BAD_ARG;
    if (fusion.rope_cos) {
        if (gated || fusion.residual || out_fp32 || !out || !fusion.rope_sin || !fusion.positions) return KB_ERR_BAD_ARG;
        if (fusion.D < 16 || fusion.D % 16 != 0 || fusion.Hq < 1 || fusion.Hkv < 1 || N != (fusion.Hq + 2 * fusion.Hkv) * fusion.D) return KB_ERR_UNSUPPORTED_SIZE;
        if (fusion.k_cache && (!fusion.v_cache || !fusion.row_ids || !fusion.block_table || !fusion.write_from || fusion.page_size < 1)) return KB_ERR_BAD_ARG;
    }
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    const __nv_bfloat16* bb = (const __nv_bfloat16*)bias;
    if (M <= 8) {
        if (gated) return launch_skinny<1, true>(xb, ldx, wb, ldw, bb, out, out_fp32, ldo, M, N, K, fusion, stream);
        return launch_skinny<1, false>(xb, ldx, wb, ldw, bb, out, out_fp32, ldo, M, N, K, fusion, stream);
    }
    if (gated) return launch_skinny<2, true>(xb, ldx, wb, ldw, bb, out, out_fp32, ldo, M, N, K, fusion, stream);
    return launch_skinny<2, false>(xb, ldx, wb, ldw, bb, out, out_fp32, ldo, M, N, K, fusion, stream);
}

KB_EXPORT int kb_gemm_skinny(const void* x, int ldx, const void* w, int ldw, const void* bias, void* out,
                             int out_fp32, int ldo, int M, int N, int K, int gated, cudaStream_t stream) {
    SkinnyFusion none = {};
    return skinny_entry(x, ldx, w, ldw, bias, out, out_fp32, ldo, M, N, K, gated, none, stream);
}

// Blocks the product of (M rows, N weight rows) is launched with: the number of partial sums
// per row that a folding epilogue writes (out_sumsq holds blocks * 16 floats).
KB_EXPORT int kb_gemm_skinny_blocks(int M, int N, int gated) {
    const int rows_out = gated ? N / 2 : N;
    int rows_per_block;
    bool three;
    skinny_grid(rows_out, !gated && M <= 8, gated != 0, rows_per_block, three);
    return (rows_out + rows_per_block - 1) / rows_per_block;
}

// Partial sums per row a scaling epilogue can add up: a folding product launched with more blocks
// than this (an output wider than 6,144 columns) cannot feed one, and the caller keeps the norm kernel.
KB_EXPORT int kb_gemm_skinny_max_sum_blocks() { return SK_SUM_BLOCKS; }

// The product with RMSNorm work in its epilogue (see the top of the file).
// in_sumsq (or null): the producer's partial sums [in_blocks, 16]; rows are scaled by
//   rsqrt(sum / in_hidden + in_eps) before bias and gate.
// residual (or null; not with gated): [M, N] fp32, row stride ldr; the result is added to it in
//   place, values[M, N] = bf16(residual * norm_w) and out_sumsq[blocks, 16] are written; out is not.
KB_EXPORT int kb_gemm_skinny_fused(const void* x, int ldx, const void* w, int ldw, const void* bias, void* out, int out_fp32,
                                   int ldo, int M, int N, int K, int gated, const float* in_sumsq, int in_blocks, int in_hidden,
                                   float in_eps, float* residual, int ldr, const void* norm_w, int norm_w_bf16, void* values,
                                   int ldv, float* out_sumsq, cudaStream_t stream) {
    SkinnyFusion fusion = {};
    fusion.in_sumsq = in_sumsq;
    fusion.in_blocks = in_blocks;
    fusion.in_inv_hidden = in_hidden > 0 ? 1.0f / (float)in_hidden : 0.0f;
    fusion.in_eps = in_eps;
    fusion.residual = residual;
    fusion.ldr = ldr;
    fusion.norm_w = norm_w;
    fusion.norm_w_bf16 = norm_w_bf16;
    fusion.values = (__nv_bfloat16*)values;
    fusion.ldv = ldv;
    fusion.out_sumsq = out_sumsq;
    return skinny_entry(x, ldx, w, ldw, bias, out, out_fp32, ldo, M, N, K, gated, fusion, stream);
}

// The q | k | v product of attention with the position encoding and the cache write in its epilogue
// (SkinnyFusion: rope).  in_sumsq (or null) as in kb_gemm_skinny_fused.  cos, sin: [max_pos, D/2] fp32
// (rotation over the whole head).  out: [M, N] bf16, of which the q columns are written; k and v go to
// the caches ([num_pages, page_size, Hkv, D] bf16; null: not written) at the slots the tokens'
// positions name in their rows' block tables.  Bad positions and pages set `flag` and are skipped.
KB_EXPORT int kb_gemm_skinny_rope(const void* x, int ldx, const void* w, int ldw, const void* bias, void* out, int ldo,
                                  int M, int N, int K, const float* in_sumsq, int in_blocks, int in_hidden, float in_eps,
                                  const float* cos_table, const float* sin_table, int max_pos, int Hq, int Hkv, int D,
                                  const int* positions, const int* row_ids, const int* block_table, int max_pages,
                                  const int* write_from, void* k_cache, void* v_cache, int page_size, int num_pages,
                                  int* flag, cudaStream_t stream) {
    SkinnyFusion fusion = {};
    fusion.in_sumsq = in_sumsq;
    fusion.in_blocks = in_blocks;
    fusion.in_inv_hidden = in_hidden > 0 ? 1.0f / (float)in_hidden : 0.0f;
    fusion.in_eps = in_eps;
    fusion.rope_cos = cos_table;
    fusion.rope_sin = sin_table;
    fusion.rope_max_pos = max_pos;
    fusion.Hq = Hq;
    fusion.Hkv = Hkv;
    fusion.D = D;
    fusion.positions = positions;
    fusion.row_ids = row_ids;
    fusion.block_table = block_table;
    fusion.max_pages = max_pages;
    fusion.write_from = write_from;
    fusion.k_cache = (__nv_bfloat16*)k_cache;
    fusion.v_cache = (__nv_bfloat16*)v_cache;
    fusion.page_size = page_size;
    fusion.num_pages = num_pages;
    fusion.flag = flag;
    if (!cos_table) return KB_ERR_NULL;
    return skinny_entry(x, ldx, w, ldw, bias, out, 0, ldo, M, N, K, 0, fusion, stream);
}
