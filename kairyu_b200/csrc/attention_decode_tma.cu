// Split-KV decode attention whose key and value tiles come in through tiled TMA copies.
//
// The cache is [pages, page_size, kv_heads, head_dim]: the 64 keys of a tile that belong to
// one KV head are page_size-long runs of rows, 2 * kv_heads * head_dim bytes apart.  A 5-D
// tensor map (64 columns, kv_heads, page_size, head_dim / 64 bands of columns, pages) lets ONE
// cp.async.bulk.tensor bring a whole run of rows with all their columns (box = 64 columns x 1 head
// x min(page_size, 64) positions x all bands x 1 page: 4 KB for 16 positions of 128 columns), so a
// tile costs a few copies instead of one per key row.  How many copies an SM can issue, not how many
// bytes they move, bounds this kernel at small pages (measured: about 50 to 75 ns a copy; with one
// 2 KB copy per band a tile of 16-position pages took 16 copies and the kernel stood at 40 GB/s an
// SM), which is why the bands, a dimension of their own with the smallest stride, travel in one
// copy.  The copies use the 128-byte swizzle; ldmatrix reads the tiles with the same XOR, which
// keeps unpadded 128-byte rows free of bank conflicts.  In shared memory a tile is
// [run of positions][band][position in the run][64 columns].
//
// Grid (rows, kv_heads, splits).  The visible tiles of a row are divided evenly over the
// splits, so a block streams a run of consecutive tiles through a ring of shared-memory
// stages: a producer warp waits for a stage to be released, looks the pages up and issues
// the copies; four consumer warps (16 keys of every tile each) wait for the stage to fill,
// compute, and release it.  The number of splits is chosen so that the grid fills the SMs
// once; a block pays its start-up latency and its epilogue once, however long the context.
// With one split the block writes the normalised output itself.  With more, partial results
// (unnormalised O, running max, running sum) go to scratch and a merge kernel combines a row's
// splits in order.  (Two other ways to combine were measured and dropped.  Letting the block that
// finishes last among a row's splits combine through global memory: its fence, its counter and its
// dependent loads all sit on the critical path of the kernel's end.  Making the splits of a (row,
// KV head) a thread-block cluster that combines through distributed shared memory: the kernel
// alone was as fast as kernel + merge, 17.2 against 17.3 us at 8 rows, but the decode step was
// 0.5 % slower, because the merge kernel's early trigger lets the output projection fetch its
// first weights while the merge runs.)  Sizes: head_dim a multiple of 64 up to 256, page_size a power of two from 8 up;
// anything else goes to the row-copy kernel of attention_mma.cuh.
//
// Variants the launcher chooses between.  At head_dim 64 a key row is 128 bytes and a copy of a run 2 KB: where
// the cache keeps the values a fixed distance behind the keys, one copy brings both (JOINED).  A grid that does
// not fit the SMs at once leaves a last wave of few blocks that run nearly alone; head_dim 64 and 128 each have a
// ring with a stage less whose blocks sit one more to an SM (TmaStages, dense_128), taken when that lets the grid
// run in fewer or fuller waves.
#include "attention_mma.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace {

constexpr int HALF_ELEMS = TILE_N * 64;  // one 64-column band of a tile: 64 rows of 128 bytes
constexpr int CONSUMER_WARPS = 4;
constexpr int KB_FLAG_TIMEOUT_DECODE = 64;  // this kernel's own bit, beside the common KB_FLAG_TIMEOUT
constexpr int MAX_SPLITS = 256;
// how a row's splits are combined (the kernel's `combine` argument)
constexpr int COMBINE_SCRATCH = 0;  // partial results to global scratch, a merge kernel follows
constexpr int COMBINE_DIRECT = 1;   // one split: the block writes the output
constexpr int MIN_TILES_PER_SPLIT = 4;   // shorter splits cost more in the combination than they save
constexpr int TMA_THREADS = (CONSUMER_WARPS + 1) * 32;  // the last warp is the producer

__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CONSUMER_WARPS * 32) : "memory"); }

// Element offset of (key of the tile, band, 8-column chunk of the band) in a tile laid out
// [run][band][position in the run][64 columns] with the 128-byte swizzle; a run has 1 << run_shift
// positions (a multiple of 8, so the swizzle's row index is the key's lowest three bits).
template <int HALVES>
__device__ __forceinline__ int tile_offset(int key, int band, int chunk, int run_shift) {
    const int row = ((((key >> run_shift) * HALVES + band) << run_shift) + (key & ((1 << run_shift) - 1)));
    return row * 64 + ((chunk ^ (key & 7)) << 3);
}

// Stages of the ring by default.  Head size 64 has a second choice, three stages: four blocks fit an SM
// then instead of three, which the launcher takes when the grid would not fit the SMs at once otherwise
// (64 rows x 8 KV heads = 512 blocks against 444 places: the 68 blocks of the second wave ran nearly
// alone and the kernel took 63 us; with 592 places it takes 45, at 91 % of the copy bandwidth).  Smaller
// grids keep four stages: a block alone on its SM needs the bytes in flight.
template <int D>
struct TmaStages {
    static constexpr int value = D <= 64 ? 4 : D <= 128 ? 3 : D <= 192 ? 2 : 3;
};

template <int D, int ST = TmaStages<D>::value>
struct TmaSmem {
    static constexpr int HALVES = D / 64;
    static constexpr int TILE_ELEMS = HALVES * HALF_ELEMS;  // K (or V) of one tile
    static constexpr int STAGE_ELEMS = 2 * TILE_ELEMS;      // K then V
    static constexpr int STAGES = ST;
    static constexpr size_t RING_BYTES = (size_t)STAGES * STAGE_ELEMS * 2;
    static constexpr size_t Q_BYTES = (size_t)16 * Tile<D>::STRIDE * 2;
    static constexpr size_t MERGE_BYTES = (size_t)(4 * 16 * (D + 8) + 2 * 4 * 16) * sizeof(float);
    static constexpr size_t BODY = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
    static constexpr size_t TOTAL = 1024 + BODY + Q_BYTES + 2 * STAGES * 8 + 16;  // slack to align the ring to 1024 bytes
};

// The tiles [t0, t1] of split `split` when the tiles [first, last] are divided evenly over `num_splits`.
__device__ __forceinline__ void split_range(int first, int last, int num_splits, int split, int& t0, int& t1, int& per) {
    const int n = last - first + 1;
    per = (n + num_splits - 1) / num_splits;
    t0 = first + split * per;
    t1 = min(t0 + per - 1, last);
}

// JOINED (head_dim 64 only): the values lie a fixed distance behind the keys in one allocation, and
// map_k has that distance as its fourth dimension in place of the bands, so that one copy brings a run
// of rows of the keys AND of the values (twice the bytes a copy; with 2 KB copies the SM's copy rate
// weighed on the kernel).  In shared memory a stage is then [run][K | V][position][64].
template <int D, bool JOINED, int ST>
__device__ __forceinline__ void
attention_decode_tma_body(const CUtensorMap& map_k, const CUtensorMap& map_v,
                          const __nv_bfloat16* __restrict__ q, int q_stride, const int* __restrict__ seq_lens,
                          const int* __restrict__ block_table, int max_pages, const int* __restrict__ decode_rows,
                          const int* __restrict__ decode_tokens, int Hq, int Hkv, int page_size, int page_shift,
                          int num_pages, float scale, int window, int num_splits, float* __restrict__ part_o,
                          float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int out_stride, int combine, int* flag) {
    using S = TmaSmem<D, ST>;
    constexpr int HALVES = S::HALVES;
    static_assert(!JOINED || HALVES == 1, "keys and values share a copy at head_dim 64 only");
    constexpr int LAY = JOINED ? 2 : HALVES;  // 64-column blocks side by side in a run of the layout
    constexpr int STAGES = S::STAGES;
    constexpr int STRIDE = Tile<D>::STRIDE;
    constexpr int CH = Tile<D>::CHUNKS;
    constexpr int KSTEPS = D / 16;
    constexpr int DTILES = D / 8;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [stage][K | V][band][64 rows][64]
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw + S::BODY);    // 16 padded rows
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + S::BODY + S::Q_BYTES);  // a stage has landed
    uint64_t* empty_bar = full_bar + STAGES;                                     // the consumers are done with a stage
    int* s_timeout = reinterpret_cast<int*>(empty_bar + STAGES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_map(&map_k);
        prefetch_map(&map_v);
#pragma unroll
        for (int st = 0; st < STAGES; ++st) {
            mbar_init(full_bar + st, 1);
            mbar_init(empty_bar + st, CONSUMER_WARPS);
        }
        *s_timeout = 0;
        fence_barrier_init();
    }
    // What follows until the waits below reads only what the host's copy of the step wrote (rows,
    // lengths, block tables) and keys and values of positions before the newest: none of it comes
    // from the kernels this one may overlap with (the products just before it, which write the
    // newest position only), so it need not wait for them.

    const int slot = blockIdx.x;
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int row = decode_rows[slot];
    const int token = decode_tokens[slot];
    const int seq_len = seq_lens[row];
    const int G = Hq / Hkv;
    const int qpos = seq_len - 1;
    const int key_lo = (window > 0 && qpos + 1 > window) ? qpos + 1 - window : 0;
    int t0, t1, per;
    split_range(key_lo / TILE_N, qpos / TILE_N, num_splits, split, t0, t1, per);
    if (seq_len < 1 || t0 > t1) {  // this split has no tile (the whole block leaves)
        pdl_wait();  // a block never ends before the kernels ahead have: those after this one count on that
        // without a merge kernel behind it, the block of an empty row writes the row's zeros
        if (combine == COMBINE_DIRECT && seq_len < 1)
            for (int idx = threadIdx.x; idx < (Hq / Hkv) * D; idx += TMA_THREADS)
                out[(size_t)token * out_stride + (size_t)(kvh * (Hq / Hkv) + idx / D) * D + idx % D] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int* table = block_table + (size_t)row * max_pages;
    const int run_shift = page_shift < 6 ? page_shift : 6;  // a copy brings min(page_size, 64) positions
    const int g = lane >> 2;
    const int tq = lane & 3;
    __syncthreads();  // the barriers are initialised

    uint32_t qf[KSTEPS][4];
    float o[DTILES][4];
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer: one copy per (K or V, 64-column band, run of rows on one page)
        const int box_rows = page_size < TILE_N ? page_size : TILE_N;
        const int runs = TILE_N / box_rows;
        const int per_tile = JOINED ? runs : 2 * runs;
        // The tile that holds the newest position is written by the kernel before this one; the tiles
        // before it are not.  Up to a ring of those go out before the wait (no stage is reused yet,
        // so nothing here waits on the consumers, who are waiting for their queries).
        const int newest_tile = qpos / TILE_N;
        int ahead = newest_tile - t0 < t1 - t0 + 1 ? newest_tile - t0 : t1 - t0 + 1;
        ahead = ahead < STAGES ? ahead : STAGES;
        if (ahead <= 0) pdl_wait();
        for (int kt = t0; kt <= t1; ++kt) {
            const int i = kt - t0;
            if (ahead > 0 && i == ahead) pdl_wait();
            const int stage = i % STAGES;
            const int use = i / STAGES;
            if (use > 0 && !mbar_wait(empty_bar + stage, (use - 1) & 1)) {
                *s_timeout = 1;
                break;
            }
            if (lane == 0) mbar_arrive_expect_tx(full_bar + stage, (uint32_t)(S::STAGE_ELEMS * sizeof(__nv_bfloat16)));
            __syncwarp();
            for (int op = lane; op < per_tile; op += 32) {
                const int is_v = JOINED ? 0 : op / runs;
                const int run = JOINED ? op : op % runs;
                const int key = kt * TILE_N + run * box_rows;
                const int page_index = key >> page_shift;
                int page = 0, within = 0;  // the reserved page stands in for rows nobody may see
                if (key < seq_len && key + box_rows > key_lo && page_index < max_pages) {
                    const int p = table[page_index];
                    if (p >= 0 && p < num_pages) {
                        page = p;
                        within = key - (page_index << page_shift);
                    }
                }
                __nv_bfloat16* dst = ring + stage * S::STAGE_ELEMS + is_v * S::TILE_ELEMS + run * LAY * box_rows * 64;
                tma_load_5d(dst, is_v ? &map_v : &map_k, 0, kvh, within, 0, page, full_bar + stage);
            }
        }
        if (ahead > 0 && t1 - t0 + 1 <= ahead) pdl_wait();  // every tile went out ahead of the wait
    } else {
        // ---------------- consumers
        pdl_wait();  // the queries come from the kernel before this one
        for (int c = threadIdx.x; c < 16 * CH; c += CONSUMER_WARPS * 32) {
            const int r = c / CH;
            const int col = (c % CH) * 8;
            const bool valid = r < G;
            const __nv_bfloat16* src = valid ? q + (size_t)token * q_stride + (size_t)(kvh * G + r) * D + col : q;
            cp_async16(sQ + r * STRIDE + col, src, valid);
        }
        cp_async_commit();
#pragma unroll
        for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
        const float sl2 = scale * LOG2E;
        cp_async_wait<0>();
        consumer_sync();  // every consumer's part of the queries is in shared memory
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int m = lane >> 3;
            const int r = (m & 1) * 8 + (lane & 7);
            const int col = ks * 16 + (m >> 1) * 8;
            ldmatrix_x4(qf[ks], sQ + r * STRIDE + col);
        }
        for (int kt = t0; kt <= t1; ++kt) {
            const int i = kt - t0;
            const int stage = i % STAGES;
            const int use = i / STAGES;
            if (!mbar_wait(full_bar + stage, use & 1)) {
                *s_timeout = 1;
                break;
            }
            __nv_bfloat16* tK = ring + stage * S::STAGE_ELEMS;
            __nv_bfloat16* tV = JOINED ? tK : tK + S::TILE_ELEMS;
            const int tile_key0 = kt * TILE_N;
            if (tile_key0 < key_lo || tile_key0 + TILE_N > seq_len) {
                // Rows nobody may see get probability 0, but 0 * NaN is NaN: clear their values
                // (a warp reads only its own 16 rows of the tile).
                for (int idx = lane; idx < 16 * HALVES * 8; idx += 32) {
                    const int r = warp * 16 + idx / (HALVES * 8);
                    const int c = idx % (HALVES * 8);
                    const int key = tile_key0 + r;
                    if (key < key_lo || key >= seq_len)
                        *reinterpret_cast<uint4*>(tV + tile_offset<LAY>(r, JOINED ? 1 : c >> 3, c & 7, run_shift)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();  // these writes stay ordered before the copy that refills the stage
                __syncwarp();
            }
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.0f;
            s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t b[4];
                const int m = lane >> 3;
                const int key = warp * 16 + (m >> 1) * 8 + (lane & 7);
                const int chunk = (ks * 2 + (m & 1)) & 7;
                ldmatrix_x4(b, tK + tile_offset<LAY>(key, JOINED ? 0 : ks >> 2, chunk, run_shift));
                mma_16816(s[0], qf[ks], b[0], b[1]);
                mma_16816(s[1], qf[ks], b[2], b[3]);
            }
            const int key_base = tile_key0 + warp * 16 + tq * 2;
            // every row of the M tile has the same query position
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key_base + nt * 8 + e;
                    const bool ok = key < seq_len && key >= key_lo;
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
                const int key = warp * 16 + (m & 1) * 8 + (lane & 7);
                const int chunk = (dp * 2 + (m >> 1)) & 7;
                ldmatrix_x4_trans(b, tV + tile_offset<LAY>(key, JOINED ? 1 : dp >> 2, chunk, run_shift));
                mma_16816(o[2 * dp], a, b[0], b[1]);
                mma_16816(o[2 * dp + 1], a, b[2], b[3]);
            }
            __syncwarp();  // every lane has read its rows of the stage
            if (lane == 0) mbar_arrive(empty_bar + stage);
        }
    }
    __syncthreads();  // producer and consumers are done with the ring before it becomes the merge buffer
    if (*s_timeout) {
        // A wait ran out.  Say so, give the copies still in flight one more bounded wait
        // (they target this block's shared memory), and leave without a result.
        if (threadIdx.x == 0) {
            if (flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_DECODE);
            for (int st = 0; st < STAGES; ++st) {
                mbar_wait(full_bar + st, 0, 1u << 10);
                mbar_wait(full_bar + st, 1, 1u << 10);
            }
        }
        return;
    }

    // combine the four consumer warps (in warp order) through shared memory
    constexpr int OSTRIDE = D + 8;
    float* sO = reinterpret_cast<float*>(smem_raw);  // [4 warps][16 rows][OSTRIDE]
    float* sM = sO + 4 * 16 * OSTRIDE;               // [4][16]
    float* sL = sM + 4 * 16;                         // [4][16]
    if (warp < CONSUMER_WARPS) {
        float l0 = l_run[0], l1 = l_run[1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
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
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += TMA_THREADS) {
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
        if (combine == COMBINE_DIRECT) {  // the only split of its row: what the merge kernel would make of it
            out[(size_t)token * out_stride + (size_t)(kvh * G + r) * D + d] = __float2bfloat16_rn(den > 0.0f ? acc / den : 0.0f);
            continue;
        }
        const size_t pidx = ((size_t)slot * Hq + (kvh * G + r)) * num_splits + split;
        part_o[pidx * D + d] = acc;
        if (d == 0) {
            part_ml[pidx * 2] = big;
            part_ml[pidx * 2 + 1] = den;
        }
    }
}

#define DECODE_TMA_PARAMS                                                                                                 \
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16* __restrict__ q, \
        int q_stride, const int* __restrict__ seq_lens, const int* __restrict__ block_table, int max_pages,                  \
        const int* __restrict__ decode_rows, const int* __restrict__ decode_tokens, int Hq, int Hkv, int page_size,          \
        int page_shift, int num_pages, float scale, int window, int num_splits, float* __restrict__ part_o,                  \
        float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int out_stride, int combine, int* flag
#define DECODE_TMA_ARGS                                                                                                     \
    map_k, map_v, q, q_stride, seq_lens, block_table, max_pages, decode_rows, decode_tokens, Hq, Hkv, page_size, page_shift, \
        num_pages, scale, window, num_splits, part_o, part_ml, out, out_stride, combine, flag

template <int D, bool JOINED, int ST>
__global__ void __launch_bounds__(TMA_THREADS) attention_decode_tma_kernel(DECODE_TMA_PARAMS) {
    attention_decode_tma_body<D, JOINED, ST>(DECODE_TMA_ARGS);
}
// head size 128 with two stages: registers held to what lets three blocks share an SM
template <>
__global__ void __launch_bounds__(TMA_THREADS, 3) attention_decode_tma_kernel<128, false, 2>(DECODE_TMA_PARAMS) {
    attention_decode_tma_body<128, false, 2>(DECODE_TMA_ARGS);
}

// grid (rows, Hq); combines the splits a row has, in split order.
__global__ void attention_decode_tma_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                  const int* __restrict__ seq_lens, const int* __restrict__ decode_rows,
                                                  const int* __restrict__ decode_tokens, __nv_bfloat16* __restrict__ out,
                                                  int out_stride, int Hq, int D, int window, int num_splits) {
    pdl_trigger();  // the product after this one may fetch its first weights meanwhile
    // rows and lengths come from the host's copy of the step: looked up ahead of the wait for the partial results
    const int slot = blockIdx.x;
    const int h = blockIdx.y;
    const int row = decode_rows[slot];
    const int token = decode_tokens[slot];
    const int seq_len = seq_lens[row];
    const int qpos = seq_len - 1;
    const int key_lo = (window > 0 && qpos + 1 > window) ? qpos + 1 - window : 0;
    int t0, t1, per;
    split_range(key_lo / TILE_N, qpos / TILE_N, num_splits, 0, t0, t1, per);
    const int tiles = seq_len < 1 ? 0 : qpos / TILE_N - key_lo / TILE_N + 1;
    const int used = (tiles + per - 1) / per;  // splits that had a tile
    const size_t base = ((size_t)slot * Hq + h) * num_splits;
    pdl_wait();
    float big = -INFINITY;
    for (int s = 0; s < used; ++s) big = fmaxf(big, part_ml[(base + s) * 2]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f, den = 0.0f;
        for (int s = 0; s < used; ++s) {
            const float ms = part_ml[(base + s) * 2];
            const float f = ms == -INFINITY ? 0.0f : exp2f(ms - big);
            acc += part_o[(base + s) * D + d] * f;
            den += part_ml[(base + s) * 2 + 1] * f;
        }
        out[(size_t)token * out_stride + (size_t)h * D + d] = __float2bfloat16_rn(den > 0.0f ? acc / den : 0.0f);
    }
}

PFN_cuTensorMapEncodeTiled g_encode = nullptr;

int get_encoder() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
    if (e != cudaSuccess) return (int)e;
    if (status != cudaDriverEntryPointSuccess || fn == nullptr) return KB_ERR_BAD_ARG;
    g_encode = (PFN_cuTensorMapEncodeTiled)fn;
    return 0;
}

// Blocks of the kernel (with its default number of stages) that fit the device at once (0 on error).
template <int D>
int resident_blocks() {
    static int cached = -1;
    if (cached >= 0) return cached;
    if (cudaFuncSetAttribute(attention_decode_tma_kernel<D, false, TmaStages<D>::value>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TmaSmem<D>::TOTAL) != cudaSuccess) return 0;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_tma_kernel<D, false, TmaStages<D>::value>, TMA_THREADS, TmaSmem<D>::TOTAL) != cudaSuccess) return 0;
    cached = sms * per_sm;
    return cached;
}

// Blocks that fit the device at once when the grid is crowded (head size 64: the three-stage ring).
int crowded_blocks_64() {
    static int cached = -1;
    if (cached >= 0) return cached;
    if (cudaFuncSetAttribute(attention_decode_tma_kernel<64, false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TmaSmem<64, 3>::TOTAL) != cudaSuccess) return 0;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_tma_kernel<64, false, 3>, TMA_THREADS, TmaSmem<64, 3>::TOTAL) != cudaSuccess) return 0;
    cached = sms * per_sm;
    return cached;
}

// Head size 128 has a second choice too: two stages, and registers held to what lets three blocks share
// an SM (444 places instead of 296).  Taken for a grid beyond 296 blocks whose whole waves of 444 hold no
// more places than its whole waves of 296 (38 to 55 rows of 8 KV heads: one wave, 55-66 us against 76-83;
// 75 to 111 rows: two waves against three, 115 us against 128 at 80 rows; 56 to 74 rows stay with two
// waves of 296: 84-98 us against 100-113).
int crowded_blocks_128() {
    static int cached = -1;
    if (cached >= 0) return cached;
    if (cudaFuncSetAttribute(attention_decode_tma_kernel<128, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TmaSmem<128, 2>::TOTAL) != cudaSuccess) return 0;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_tma_kernel<128, false, 2>, TMA_THREADS, TmaSmem<128, 2>::TOTAL) != cudaSuccess) return 0;
    cached = sms * per_sm;
    return cached;
}

bool dense_128(long long blocks) {
    const long long usual = resident_blocks<128>(), dense = crowded_blocks_128();
    if (usual <= 0 || dense <= 0 || blocks <= usual) return false;
    return (blocks + dense - 1) / dense * dense <= (blocks + usual - 1) / usual * usual;
}

int resident_blocks_for(int D) {
    switch (D) {
        case 64: return resident_blocks<64>();
        case 128: return resident_blocks<128>();
        case 192: return resident_blocks<192>();
        case 256: return resident_blocks<256>();
        default: return 0;
    }
}

template <int D, bool JOINED, int ST = TmaStages<D>::value>
int launch(const CUtensorMap* mk, const CUtensorMap* mv, const __nv_bfloat16* q, int q_stride, const int* seq_lens,
           const int* block_table, int max_pages, const int* decode_rows, const int* decode_tokens, int num_rows, int Hq,
           int Hkv, int page_size, int num_pages, float scale, int window, int num_splits, float* part_o, float* part_ml,
           __nv_bfloat16* out, int out_stride, int combine, int* flag, cudaStream_t stream) {
    const size_t smem = TmaSmem<D, ST>::TOTAL;
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<D, JOINED, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;  // page_size is a power of two here
    dim3 grid(num_rows, Hkv, num_splits);
    kb_launch(attention_decode_tma_kernel<D, JOINED, ST>, dim3(grid), dim3(TMA_THREADS), smem, stream, *mk, *mv, q, q_stride, seq_lens,
              block_table, max_pages, decode_rows, decode_tokens, Hq, Hkv, page_size, shift, num_pages, scale,
              window, num_splits, part_o, part_ml, out, out_stride, combine, flag);
    return kb_launch_result();
}

}  // namespace

// 1 when (head_dim, page_size) fit this kernel.
KB_EXPORT int kb_attention_decode_tma_supported(int D, int page_size) {
    if (D != 64 && D != 128 && D != 192 && D != 256) return 0;
    if (page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
    return 1;
}

// Splits this kernel should be launched with for `num_rows` rows of up to `max_seq_len`
// keys: as many as let rows * kv_heads * splits blocks be resident at once, at least 1, at
// most one per four 64-key tiles and at most 256.  Returns a negative KB_ERR_* code on error.
KB_EXPORT int kb_attention_decode_tma_splits(int num_rows, int Hkv, int D, int max_seq_len) {
    if (num_rows < 1 || Hkv < 1 || max_seq_len < 1) return KB_ERR_BAD_ARG;
    const int resident = resident_blocks_for(D);
    if (resident <= 0) return KB_ERR_UNSUPPORTED_SIZE;
    const long long pairs = (long long)num_rows * Hkv;
    long long splits = resident / pairs;
    const int tiles = (max_seq_len + TILE_N - 1) / TILE_N;
    const int worthwhile = (tiles + MIN_TILES_PER_SPLIT - 1) / MIN_TILES_PER_SPLIT;
    if (pairs > resident) {
        // More (row, KV head) pairs than places: with one block a pair, the blocks beyond the first wave
        // run nearly alone (304 pairs on 296 places took 76 us where 288 take 50).  Two splits a pair make
        // the last wave a smaller share: in units of a whole pair's time the kernel takes about
        // ceil(2 * pairs / places) / 2, and the merge launch and the second start a tenth.  Taken where
        // that gains 15 % or more on ceil(pairs / places): measured 8-9 % on the kernel at 38 to 48 rows of
        // 8 KV heads (head size 128), nothing or a loss outside that range and with more splits.
        const int places = D == 64 ? crowded_blocks_64() : resident;
        if (places <= 0) return KB_ERR_UNSUPPORTED_SIZE;
        if (D == 128 && dense_128(pairs)) return 1;  // whole waves of three blocks an SM
        const double whole = (double)((pairs + places - 1) / places);
        const double halves = (double)((pairs * 2 + places - 1) / places) / 2 + 0.1;
        return (worthwhile >= 2 && halves < 0.85 * whole) ? 2 : 1;
    }
    if (splits > worthwhile) splits = worthwhile;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits < 1) splits = 1;
    return (int)splits;
}

// Writes a 128-byte tensor map (host memory, 64-byte aligned) for a bf16 cache
// [num_pages, page_size, kv_heads, head_dim] with the given strides in elements (head_dim
// contiguous).  ``bands`` = 0: four dimensions (head_dim, kv_heads, page_size, pages), boxes of 64
// columns x 1 head x min(page_size, 64) positions x 1 page (the prefill kernel's copies, one per
// 64-column band).  ``bands`` = 1: five dimensions (64 columns, kv_heads, page_size, head_dim / 64
// bands, pages), boxes that take every band at once (this kernel's copies).  128-byte swizzle.
KB_EXPORT int kb_attention_encode_cache_map(void* map_out, const void* base, long long num_pages, int page_size, int Hkv, int D,
                                            long long stride_page, long long stride_pos, long long stride_head, int bands) {
    if (!map_out || !base) return KB_ERR_NULL;
    if (((uintptr_t)map_out % 64) != 0 || ((uintptr_t)base % 16) != 0) return KB_ERR_BAD_ARG;
    if (!kb_attention_decode_tma_supported(D, page_size) || num_pages < 1 || Hkv < 1) return KB_ERR_UNSUPPORTED_SIZE;
    if ((stride_page * 2) % 16 != 0 || (stride_pos * 2) % 16 != 0 || (stride_head * 2) % 16 != 0) return KB_ERR_UNSUPPORTED_SIZE;
    const int rc = get_encoder();
    if (rc != 0) return rc;
    const cuuint32_t box_rows = (cuuint32_t)(page_size < TILE_N ? page_size : TILE_N);
    CUresult r;
    if (bands) {
        cuuint64_t dims[5] = {64, (cuuint64_t)Hkv, (cuuint64_t)page_size, (cuuint64_t)(D / 64), (cuuint64_t)num_pages};
        cuuint64_t strides[4] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_pos * 2, 128, (cuuint64_t)stride_page * 2};
        cuuint32_t box[5] = {64, 1, box_rows, (cuuint32_t)(D / 64), 1};
        cuuint32_t elem[5] = {1, 1, 1, 1, 1};
        r = g_encode((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)Hkv, (cuuint64_t)page_size, (cuuint64_t)num_pages};
        cuuint64_t strides[3] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_pos * 2, (cuuint64_t)stride_page * 2};
        cuuint32_t box[4] = {64, 1, box_rows, 1};
        cuuint32_t elem[4] = {1, 1, 1, 1};
        r = g_encode((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// A map over keys AND values of a cache whose values lie `gap` elements behind its keys, with the same
// shape and strides (head_dim 64): five dimensions (64 columns, kv_heads, page_size, keys | values, pages),
// boxes of 1 head x min(page_size, 64) positions of both.  128-byte swizzle.
KB_EXPORT int kb_attention_encode_joined_map(void* map_out, const void* base_k, long long gap, long long num_pages, int page_size,
                                             int Hkv, int D, long long stride_page, long long stride_pos, long long stride_head) {
    if (!map_out || !base_k) return KB_ERR_NULL;
    if (((uintptr_t)map_out % 64) != 0 || ((uintptr_t)base_k % 16) != 0) return KB_ERR_BAD_ARG;
    if (D != 64 || !kb_attention_decode_tma_supported(D, page_size) || num_pages < 1 || Hkv < 1) return KB_ERR_UNSUPPORTED_SIZE;
    if ((stride_page * 2) % 16 != 0 || (stride_pos * 2) % 16 != 0 || (stride_head * 2) % 16 != 0) return KB_ERR_UNSUPPORTED_SIZE;
    if (gap <= 0 || (gap * 2) % 16 != 0 || gap * 2 >= (1ll << 40)) return KB_ERR_UNSUPPORTED_SIZE;  // a stride has 40 bits
    const int rc = get_encoder();
    if (rc != 0) return rc;
    const cuuint32_t box_rows = (cuuint32_t)(page_size < TILE_N ? page_size : TILE_N);
    cuuint64_t dims[5] = {64, (cuuint64_t)Hkv, (cuuint64_t)page_size, 2, (cuuint64_t)num_pages};
    cuuint64_t strides[4] = {(cuuint64_t)stride_head * 2, (cuuint64_t)stride_pos * 2, (cuuint64_t)gap * 2, (cuuint64_t)stride_page * 2};
    cuuint32_t box[5] = {64, 1, box_rows, 2, 1};
    cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult r = g_encode((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base_k), dims, strides, box,
                                elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// map_k, map_v: host pointers to tensor maps made by kb_attention_encode_cache_map with bands = 1; with
// `joined` (head_dim 64 only), map_k is a map of kb_attention_encode_joined_map and map_v is not read.
// num_splits: any value from 1 up (kb_attention_decode_tma_splits gives a good one).
// part_o: [rows, Hq, splits, D] fp32; part_ml: [rows, Hq, splits, 2] fp32 (scratch; only read
// and written with more than one split).
KB_EXPORT int kb_attention_decode_tma(const void* map_k, const void* map_v, const void* q, int q_stride, void* out, int out_stride,
                                      const int* seq_lens, const int* block_table, int max_pages, const int* decode_rows,
                                      const int* decode_tokens, int num_rows, int Hq, int Hkv, int D, int page_size, int num_pages,
                                      float scale, int window, int num_splits, float* part_o, float* part_ml, int joined, int* flag,
                                      cudaStream_t stream) {
    if (num_rows == 0) return 0;
    if (joined && D != 64) return KB_ERR_UNSUPPORTED_SIZE;
    if (joined) map_v = map_k;
    if (!map_k || !map_v || !q || !out || !seq_lens || !block_table || !decode_rows || !decode_tokens) return KB_ERR_NULL;
    const int combine = num_splits == 1 ? COMBINE_DIRECT : COMBINE_SCRATCH;
    if (combine == COMBINE_SCRATCH && (!part_o || !part_ml)) return KB_ERR_NULL;
    if (out_stride % 2 != 0) return KB_ERR_BAD_ARG;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16 || Hkv > 65535 || num_splits < 1 || num_splits > MAX_SPLITS) return KB_ERR_BAD_ARG;
    if (q_stride % 8 != 0) return KB_ERR_BAD_ARG;
    if (!kb_attention_decode_tma_supported(D, page_size)) return KB_ERR_UNSUPPORTED_SIZE;
    const CUtensorMap* mk = (const CUtensorMap*)map_k;
    const CUtensorMap* mv = (const CUtensorMap*)map_v;
    int rc;
#define ARGS mk, mv, (const __nv_bfloat16*)q, q_stride, seq_lens, block_table, max_pages, decode_rows, decode_tokens, num_rows, Hq, \
             Hkv, page_size, num_pages, scale, window, num_splits, part_o, part_ml, (__nv_bfloat16*)out, out_stride, combine, flag, stream
    switch (D) {
        case 64: {
            // a grid that four-stage blocks cannot hold at once runs with three stages, four blocks an SM
            const bool crowded = (long long)num_rows * Hkv * num_splits > resident_blocks<64>();
            if (crowded) rc = joined ? launch<64, true, 3>(ARGS) : launch<64, false, 3>(ARGS);
            else rc = joined ? launch<64, true>(ARGS) : launch<64, false>(ARGS);
            break;
        }
        case 128: {
            const long long blocks = (long long)num_rows * Hkv * num_splits;
            if (dense_128(blocks)) rc = launch<128, false, 2>(ARGS);
            else rc = launch<128, false>(ARGS);
            break;
        }
        case 192: rc = launch<192, false>(ARGS); break;
        default: rc = launch<256, false>(ARGS); break;
    }
#undef ARGS
    if (rc != 0 || combine != COMBINE_SCRATCH) return rc;
    dim3 grid(num_rows, Hq);
    kb_launch(attention_decode_tma_merge_kernel, dim3(grid), dim3(128), 0, stream, part_o, part_ml, seq_lens, decode_rows,
              decode_tokens, (__nv_bfloat16*)out, out_stride, Hq, D, window, num_splits);
    return kb_launch_result();
}

// Launches kb_attention_decode_tma makes for this many splits: 1, or 2 when a merge kernel follows.
KB_EXPORT int kb_attention_decode_tma_launches(int num_splits) { return num_splits > 1 ? 2 : 1; }
