// Flash attention over the paged cache for rows that carry several tokens, on the
// 5th-generation tensor cores (kairyu/models/attention.py:203-240 is the arithmetic):
//
//     S = Q K^T * scale (causal, optional window),  P = softmax rows online,  O = P V.
//
// Three ways to spread a step's query tiles over the device, chosen on the host:
//  * one tile of 128 queries a block, the longest first (later tiles of a portion see more keys),
//    when the blocks fit the device at once, or are far too many to;
//  * two tiles a block, tile T-1-y and then tile y, when one tile a block would not all run at once
//    but two a block do (a prompt of 2,048 tokens: 16 tiles x 32 heads): every block then does the
//    same work (34 key tiles) instead of the longest walking its 32 key tiles alone at the end
//    (2,048 tokens: 63 -> 59 us; at 8,192 tokens equal blocks would fill their last wave badly);
//  * several blocks a tile, each with a share of the tile's keys, when the tiles alone would leave
//    most of the device idle (a 512-token portion at the end of 8,192 tokens is 128 tiles x heads:
//    312 -> 102 us); the blocks leave unnormalised O, their reference maximum and their sum in
//    fp32 scratch, and a second kernel combines them in split order.
// Long portions of head_dim 128 go to a second kernel further down, which walks two tiles side by side.
// For a tile the block walks the keys it may see in tiles of 64.  Roles (192 threads):
//   warp 0     producer: TMA copies of the Q tile (2-D map over the packed qkv rows) and of
//              every K and V tile (a map over the cache: a copy brings a page's run of rows
//              for one KV head), two stages ahead of their use;
//   warp 1     one thread issues tcgen05.mma: S = Q K^T into one of two buffers of 64 TMEM
//              columns, O += P V into head_dim TMEM columns.  Q K^T runs two tiles ahead of
//              P V, so the softmax warps never wait for their S;
//   warps 2-5  softmax: thread r owns query row r.  It reads its row of S from TMEM
//              (tcgen05.ld), so the row maximum and sum need no shuffles; writes P as bf16
//              pairs back into tensor memory over its row of S (tcgen05.st), from where the
//              tensor core reads it as the A operand of P V; and rescales O in TMEM only when
//              the row maximum has grown by more than 2^8 since the reference it scales by
//              (P stays below 256, sums stay exact enough in fp32).  Only then does it wait
//              for the P V before to finish; otherwise it goes straight on to the next S.
// V is the B operand of O += P V with its N index (the head dimension) contiguous: an
// MN-major operand, read straight from the [key][dim] rows the cache holds.
// Two blocks share an SM (2 x 256 TMEM columns, 2 x 97 KB of shared memory), so one block's
// softmax overlaps the other's products.
//
// How many copies an SM can issue bounds this kernel before the tensor cores do (about 50 to
// 75 ns a copy were measured; a 64-key tile of 16-position pages and 128 columns is 16 copies of
// 2 KB with one copy per 64-column band, 1 us a tile, against 0.28 us of products).  So for
// head_dim 128 and pages of 16 positions or more the copies of V take both bands at once
// (`merged`: a 5-D map whose band dimension has the smallest stride; 12 copies a tile).  A V tile
// then lies in shared memory as [run of positions][band][position][64 columns]; P V, whose steps
// are 16 keys anyway, only takes other strides.  K keeps a copy per band: as a K-major operand it
// needs its 8-row groups evenly spaced over all 64 keys, and issuing Q K^T run by run instead
// (N = 16) cost more on the tensor cores than the copies saved (104 against 71 us for 2,048 tokens).
//
// Every wait on an mbarrier is bounded: a role that gives up raises KB_FLAG_TIMEOUT, lets the
// other roles leave through a shared abort word, and the block frees its TMEM and returns.
// Sizes: head_dim 64 or 128, page_size a power of two from 8 up; others go to the mma.sync
// kernel of attention_mma.cuh.
#include "umma.cuh"

#define FA_THREADS 192
#define FA_BM 128
#define FA_BN 64
#define FA_STAGES 2
#define FA_LOG2E 1.4426950408889634f
#define FA_RESCALE_STEP 8.0f
#define KB_FLAG_MISALIGNED 32
#define KB_FLAG_TIMEOUT_PREFILL 128  // this kernel's own bit, beside the common KB_FLAG_TIMEOUT

// 2^x, flushing denormals: one MUFU instruction (exp2f adds range handling around it).
__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Two fp32 operations in one instruction (sm_100 packs two floats in a 64-bit register).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n"
        : "=l"(d)
        : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)), "l"(*reinterpret_cast<uint64_t*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <int D>
struct FaCfg {
    static constexpr int BANDS = D / 64;                 // 64-column (128-byte) bands of a row
    static constexpr int Q_BAND = FA_BM * 128;           // bytes of one band of the Q tile
    static constexpr int KV_BAND = FA_BN * 128;          // bytes of one band of a K or V tile
    static constexpr int Q_BYTES = BANDS * Q_BAND;
    static constexpr int KV_BYTES = BANDS * KV_BAND;
    static constexpr int OFF_K = Q_BYTES;
    static constexpr int OFF_V = OFF_K + FA_STAGES * KV_BYTES;
    static constexpr int OFF_BAR = OFF_V + FA_STAGES * KV_BYTES;
    static constexpr int NUM_BARS = 1 + 4 * FA_STAGES + 2 + 2 + 2 + 1;
    static constexpr size_t SMEM = OFF_BAR + NUM_BARS * 8 + 16;
    static constexpr int S_COL = 0;          // two S buffers of FA_BN columns each; P (bf16 pairs) overwrites the first half of its S
    static constexpr int O_COL = 2 * FA_BN;
    static constexpr int TMEM_COLUMNS = 256;
    static constexpr int BLOCKS_PER_SM = 2;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, FaCfg<D>::BLOCKS_PER_SM)
attention_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int out_stride,
                             const int* __restrict__ qo_indptr, const int* __restrict__ seq_lens,
                             const int* __restrict__ block_table, int max_pages, const int* __restrict__ tile_rows,
                             const int* __restrict__ tile_starts, int num_tiles, int Hq, int Hkv, int page_size, int page_shift,
                             int num_pages, float scale, int window, int merged, int paired, int splits, float* __restrict__ part_o,
                             float* __restrict__ part_ml, int* flag) {
    using Cfg = FaCfg<D>;
    constexpr int BANDS = Cfg::BANDS;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* sQ = smem;
    unsigned char* sK = smem + Cfg::OFF_K;
    unsigned char* sV = smem + Cfg::OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = k_full + FA_STAGES;
    uint64_t* k_empty = v_full + FA_STAGES;
    uint64_t* v_empty = k_empty + FA_STAGES;
    uint64_t* s_full = v_empty + FA_STAGES;  // one per S buffer
    // p_full and pv_done: two each, used in turn by the key tiles (tile g uses [g % 2]).  The softmax may
    // be a tile ahead of the thread that issues the products (it needs no P V to go on), and one barrier
    // whose phase is told by its parity cannot be two phases ahead of who waits on it.
    uint64_t* p_full = s_full + 2;
    uint64_t* pv_done = p_full + 2;
    uint64_t* q_empty = pv_done + 2;  // every Q K^T of a query tile has read the queries' buffer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < FA_STAGES; ++s) {
            mbar_init(k_full + s, 1);
            mbar_init(v_full + s, 1);
            mbar_init(k_empty + s, 1);
            mbar_init(v_empty + s, 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_full + 1, 1);
        mbar_init(p_full, 4);
        mbar_init(p_full + 1, 4);
        mbar_init(pv_done, 1);
        mbar_init(pv_done + 1, 1);
        mbar_init(q_empty, 1);
        *abort_word = 0;
        if ((smem_addr(smem) & 1023u) != 0) {  // the swizzled layouts below assume it
            if (flag) atomicOr(flag, KB_FLAG_MISALIGNED);
            *abort_word = 1;
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    // The block's two tiles: a long one first (later tiles of a portion see more keys), then the short
    // one from the other end of the list.  Barrier phases run on through both: `g` counts key tiles
    // since the block began.
    const int h = blockIdx.x;
    const int kvh = h / (Hq / Hkv);
    const int num_parts = (paired && (int)blockIdx.y != num_tiles - 1 - (int)blockIdx.y) ? 2 : 1;
    // Layout of a V tile: rows of a band lie `run_rows` x 128 bytes from the next band's, and a run
    // of positions BANDS x run_rows x 128 bytes from the next run (not merged: one run of 64, as K).
    const int box_rows = page_size < FA_BN ? page_size : FA_BN;
    const int run_rows = merged ? box_rows : FA_BN;
    const int band_bytes = run_rows * 128;
    const int run_bytes = BANDS * band_bytes;

    struct TileInfo {
        int tile, row, q0, tok0, rows_here, first_pos, last_pos, key_end, key_lo, first_kt, num_kt;
    };
    auto tile_info = [&](int part) {
        TileInfo t;
        const int tile = part == 0 ? num_tiles - 1 - (int)blockIdx.y : (int)blockIdx.y;
        t.tile = tile;
        t.row = tile_rows[tile];
        t.q0 = tile_starts[tile];
        t.tok0 = qo_indptr[t.row];
        const int chunk_len = qo_indptr[t.row + 1] - t.tok0;
        const int seq_len = seq_lens[t.row];
        const int chunk_pos = seq_len - chunk_len;  // absolute position of the portion's first token
        t.rows_here = min(FA_BM, chunk_len - t.q0);
        t.first_pos = chunk_pos + t.q0;
        t.last_pos = t.first_pos + t.rows_here - 1;
        t.key_end = t.last_pos + 1;  // causal bound of the tile (<= seq_len)
        t.key_lo = (window > 0 && t.first_pos + 1 > window) ? t.first_pos + 1 - window : 0;
        t.first_kt = t.key_lo / FA_BN;
        t.num_kt = (t.key_end - 1) / FA_BN - t.first_kt + 1;
        if (splits > 1) {
            // this block's share of the tile's keys: split z takes key tiles [z * per, (z + 1) * per); a
            // short tile leaves the last splits without any (num_kt <= 0: the block only says so)
            const int per = (t.num_kt + splits - 1) / splits;
            const int begin = (int)blockIdx.z * per;
            const int end = min(begin + per, t.num_kt);
            t.first_kt += begin;
            t.num_kt = end - begin;
        }
        return t;
    };

    if (*abort_word) {
        // fall through to the common exit
    } else if (warp == 0) {
        // ---------------- producer
        const int runs = FA_BN / box_rows;
        const int per_k = BANDS * runs;                     // copies of a K tile
        const int per_v = merged ? runs : BANDS * runs;     // copies of a V tile
        bool ok = true;
        int g0 = 0;
        for (int part = 0; part < num_parts && ok; ++part) {
            const TileInfo t = tile_info(part);
            if (t.num_kt <= 0) break;  // a split without keys (splits > 1: one part a block)
            // the queries' buffer is free once every Q K^T of the tile before has read it
            if (part > 0 && !mbar_wait(q_empty, (part - 1) & 1, abort_word)) {
                if (lane == 0 && !*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
                *abort_word = 1;
                break;
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
                for (int band = 0; band < BANDS; ++band)
                    tma_load_2d_plain(sQ + band * Cfg::Q_BAND, &map_q, h * D + band * 64, t.tok0 + t.q0, q_full);
            }
            const int* table = block_table + (size_t)t.row * max_pages;
            for (int j = 0; j < t.num_kt && ok; ++j) {
                const int g = g0 + j;
                const int st = g % FA_STAGES;
                const int use = g / FA_STAGES;
#pragma unroll
                for (int is_v = 0; is_v < 2; ++is_v) {
                    // K's slot is free once Q K^T of the tile that used it is done, V's once its P V is done
                    if (use > 0 && !mbar_wait((is_v ? v_empty : k_empty) + st, (use - 1) & 1, abort_word)) {
                        if (lane == 0 && !*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
                        *abort_word = 1;
                        ok = false;
                        break;
                    }
                    uint64_t* bar = (is_v ? v_full : k_full) + st;
                    if (lane == 0) mbar_arrive_expect_tx(bar, Cfg::KV_BYTES);
                    __syncwarp();
                    for (int op = lane; op < (is_v ? per_v : per_k); op += 32) {
                        const int band = op / runs;  // 0 when the copy takes every band
                        const int run = op % runs;
                        const int key = (t.first_kt + j) * FA_BN + run * box_rows;
                        const int page_index = key >> page_shift;
                        int page = 0, within = 0;  // the reserved page stands in for rows nobody may see
                        if (key < t.key_end && key + box_rows > t.key_lo && page_index < max_pages) {
                            const int p = table[page_index];
                            if (p >= 0 && p < num_pages) {
                                page = p;
                                within = key - (page_index << page_shift);
                            }
                        }
                        unsigned char* tile_base = (is_v ? sV : sK) + st * Cfg::KV_BYTES;
                        if (is_v && merged)
                            tma_load_5d_plain(tile_base + run * run_bytes, &map_v, 0, kvh, within, 0, page, bar);
                        else
                            tma_load_4d_plain(tile_base + band * Cfg::KV_BAND + run * box_rows * 128, is_v ? &map_v : &map_k, band * 64, kvh, within, page, bar);
                    }
                }
            }
            g0 += t.num_kt;
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc(FA_BN);
            constexpr uint32_t idesc_pv = umma_idesc_b_mn(D);
            // Descriptors differ only in their start address (bits 0-13, in 16-byte units): build
            // one of each kind and add offsets.
            const uint64_t q_desc = umma_desc_sw128(smem_addr(sQ));
            const uint64_t k_desc = umma_desc_sw128(smem_addr(sK));
            const uint64_t v_desc = umma_desc_mn_sw128(smem_addr(sV), (uint32_t)band_bytes, 1024);
            // Where the 16 keys of a P V step lie in a V tile, worked out once: this thread shares its
            // scheduler with softmax warps, and every instruction it spends between two products is a
            // product issued later (divisions by the run length in the loop held the products back).
            uint64_t v_step[FA_BN / 16];
#pragma unroll
            for (int ks = 0; ks < FA_BN / 16; ++ks) {
                const int key = ks * 16;
                v_step[ks] = (uint64_t)(((key / run_rows) * run_bytes + (key % run_rows) * 128) >> 4);
            }
            bool ok = true;
            auto give_up = [&]() {
                if (!*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
                *abort_word = 1;
                ok = false;
            };
            // S[g % 2] = Q K_g^T; releases K's slot and tells the softmax warps
            auto issue_qk = [&](int g, bool last_of_tile) {
                const int st = g % FA_STAGES;
                const uint64_t k_tile = k_desc + (uint64_t)((st * Cfg::KV_BYTES) >> 4);
#pragma unroll
                for (int band = 0; band < BANDS; ++band)
#pragma unroll
                    for (int k = 0; k < 4; ++k)  // 16 of the head dimension = 32 bytes along the swizzled row
                        umma_bf16(tmem_base + Cfg::S_COL + (g & 1) * FA_BN, q_desc + (uint64_t)((band * Cfg::Q_BAND + k * 32) >> 4),
                                  k_tile + (uint64_t)((band * Cfg::KV_BAND + k * 32) >> 4), idesc_qk, (band > 0 || k > 0) ? 1u : 0u);
                umma_commit(k_empty + st);
                umma_commit(s_full + (g & 1));
                if (last_of_tile) umma_commit(q_empty);  // the queries' buffer may take the next tile's
            };
            int g0 = 0;
            for (int part = 0; part < num_parts && ok; ++part) {
                const int num_kt = tile_info(part).num_kt;
                if (num_kt <= 0) break;  // a split without keys
                // Q K^T runs two key tiles ahead of P V.  (The two S buffers are free here: the products that
                // read the tile before's last P were issued before these, and the tensor pipe keeps the order.)
                if (!mbar_wait(q_full, part & 1, abort_word) || !mbar_wait(k_full + g0 % FA_STAGES, (g0 / FA_STAGES) & 1, abort_word)) give_up();
                if (ok) {
                    tc_fence_after();
                    issue_qk(g0, num_kt == 1);
                }
                if (ok && num_kt > 1) {
                    if (!mbar_wait(k_full + (g0 + 1) % FA_STAGES, ((g0 + 1) / FA_STAGES) & 1, abort_word)) give_up();
                    if (ok) {
                        tc_fence_after();
                        issue_qk(g0 + 1, num_kt == 2);
                    }
                }
                for (int j = 0; j < num_kt && ok; ++j) {
                    const int g = g0 + j;
                    const int st = g % FA_STAGES;
                    if (!mbar_wait(p_full + (g & 1), (g >> 1) & 1, abort_word) || !mbar_wait(v_full + st, (g / FA_STAGES) & 1, abort_word)) {
                        give_up();
                        break;
                    }
                    tc_fence_after();
                    const uint64_t v_tile = v_desc + (uint64_t)((st * Cfg::KV_BYTES) >> 4);
#pragma unroll
                    for (int ks = 0; ks < FA_BN / 16; ++ks)  // 16 keys: 8 columns of P in tensor memory, 16 rows of V
                        umma_bf16_a_tmem(tmem_base + Cfg::O_COL, tmem_base + Cfg::S_COL + (g & 1) * FA_BN + ks * 8,
                                         v_tile + v_step[ks], idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(v_empty + st);  // the slot may be refilled once these products have read it
                    umma_commit(pv_done + (g & 1));
                    if (j + 2 < num_kt) {
                        // the softmax warps hold S_g in registers (they have written P_g): its buffer takes tile g + 2
                        if (!mbar_wait(k_full + st, ((g + 2) / FA_STAGES) & 1, abort_word)) {
                            give_up();
                            break;
                        }
                        tc_fence_after();
                        issue_qk(g + 2, j + 3 == num_kt);
                    }
                }
                g0 += num_kt;
            }
        }
    } else {
        // ---------------- softmax and epilogue: thread r owns query row r
        const int quarter = warp & 3;  // the TMEM lanes this warp may touch
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int soft_tid = threadIdx.x - 64;  // 0..127
        const float sl2 = scale * FA_LOG2E;
        bool ok = true;
        int g0 = 0;
        for (int part = 0; part < num_parts && ok; ++part) {
            const TileInfo t = tile_info(part);
            const int num_kt = t.num_kt, first_kt = t.first_kt, first_pos = t.first_pos, last_pos = t.last_pos, key_end = t.key_end;
            const bool valid = r < t.rows_here;
            // with the keys split over blocks: where this block's unnormalised O, reference maximum and sum go
            const size_t part_slot = (((size_t)blockIdx.z * num_tiles + t.tile) * FA_BM + r) * Hq + h;
            if (num_kt <= 0) {
                if (valid) {
                    part_ml[part_slot * 2] = -INFINITY;
                    part_ml[part_slot * 2 + 1] = 0.0f;
                }
                break;
            }
            const int pos = valid ? first_pos + r : last_pos;
            const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            const int lo_last = (window > 0 && last_pos + 1 > window) ? last_pos + 1 - window : 0;
            float m_ref = -INFINITY;  // the maximum the row's P and O are scaled by
            float l = 0.0f;
            for (int j = 0; j < num_kt; ++j) {
                const int g = g0 + j;
                const int key0 = (first_kt + j) * FA_BN;
                if (!mbar_wait(s_full + (g & 1), (g >> 1) & 1, abort_word)) { ok = false; break; }
                tc_fence_after();
                uint32_t raw[2][32];
                tmem_load32_nowait(lane_base + Cfg::S_COL + (g & 1) * FA_BN, raw[0]);
                tmem_load32_nowait(lane_base + Cfg::S_COL + (g & 1) * FA_BN + 32, raw[1]);
                tmem_wait_ld();
                // Work on the raw scores: the row maximum is taken before the scale (scale > 0), and
                // scale and reference enter the exponent's argument as one fused multiply-add.
                float tt[FA_BN];
#pragma unroll
                for (int c = 0; c < FA_BN; ++c) tt[c] = __uint_as_float(raw[c >> 5][c & 31]);
                if (key0 + FA_BN - 1 > first_pos || key0 < lo_last) {  // the diagonal or the window's edge crosses this tile
#pragma unroll
                    for (int c = 0; c < FA_BN; ++c) {
                        const int key = key0 + c;
                        tt[c] = (key <= pos && key >= lo) ? tt[c] : -INFINITY;
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < FA_BN; c += 8) {
                    mx4[0] = max3(mx4[0], tt[c], tt[c + 1]);
                    mx4[1] = max3(mx4[1], tt[c + 2], tt[c + 3]);
                    mx4[2] = max3(mx4[2], tt[c + 4], tt[c + 5]);
                    mx4[3] = max3(mx4[3], tt[c + 6], tt[c + 7]);
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;  // -inf stays -inf
                float alpha = 1.0f;
                if (m_ref == -INFINITY) {
                    m_ref = mx;  // nothing accumulated for this row yet
                } else if (mx > m_ref + FA_RESCALE_STEP) {
                    alpha = exp2f(m_ref - mx);
                    m_ref = mx;
                }
                // The softmax does not wait for P V of the tile before: only a rescale of O needs it complete,
                // and that is rare.  Every phase of the two pv_done barriers is still observed, in order and
                // two tiles late (a parity wait cannot tell a phase from the one two before it); a query
                // tile's last two phases are observed by its epilogue.
                if (j > 1 && !mbar_wait(pv_done + (g & 1), ((g - 2) >> 1) & 1, abort_word)) { ok = false; break; }
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    if (j > 0 && !mbar_wait(pv_done + ((g - 1) & 1), ((g - 1) >> 1) & 1, abort_word)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t o[32];
                        tmem_load32_nowait(lane_base + Cfg::O_COL + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_store32(lane_base + Cfg::O_COL + c * 32, o);
                    }
                    tmem_wait_st();
                    l *= alpha;
                }
                const float neg_base = m_ref == -INFINITY ? 0.0f : -m_ref;
                const float2 scale2 = make_float2(sl2, sl2);
                const float2 base2 = make_float2(neg_base, neg_base);
                float2 sum2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
                uint32_t packed[FA_BN / 2];
#pragma unroll
                for (int c = 0; c < FA_BN; c += 2) {
                    const float2 arg = ffma2(make_float2(tt[c], tt[c + 1]), scale2, base2);  // (-inf) * scale + base = -inf
                    // (A cubic for 2^x on the FMA pipes for every fourth pair, to spare the special-function unit,
                    // made the kernel slower, 54 -> 57 us at 2,048 tokens: the exponentials are not what it waits for.)
                    const float2 p = make_float2(ex2_ftz(arg.x), ex2_ftz(arg.y));
                    sum2[(c >> 1) & 1] = fadd2(sum2[(c >> 1) & 1], p);
                    __nv_bfloat162 pair = __floats2bfloat162_rn(p.x, p.y);
                    packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                }
                const float sum = (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
                l += sum;
                // P_g takes the place of the first half of S_g: this thread's own row, which it holds in registers
                tmem_store32(lane_base + Cfg::S_COL + (g & 1) * FA_BN, packed);
                tmem_wait_st();
                if (key0 + FA_BN > key_end) {
                    // Keys beyond the last query have probability 0, but 0 * NaN is NaN and what lies
                    // beyond a request's length may be anything: clear those rows of V.
                    const int st = g % FA_STAGES;
                    if (!mbar_wait(v_full + st, (g / FA_STAGES) & 1, abort_word)) { ok = false; break; }
                    unsigned char* v_tile = sV + st * Cfg::KV_BYTES;
                    for (int idx = soft_tid; idx < FA_BN * BANDS * 8; idx += 128) {
                        const int vr = idx / (BANDS * 8);
                        const int c = idx % (BANDS * 8);
                        if (key0 + vr >= key_end)
                            *reinterpret_cast<uint4*>(v_tile + (vr / run_rows) * run_bytes + (c >> 3) * band_bytes + (vr % run_rows) * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + (g & 1));
            }
            if (ok && num_kt > 1 && !mbar_wait(pv_done + ((g0 + num_kt - 2) & 1), ((g0 + num_kt - 2) >> 1) & 1, abort_word)) ok = false;
            if (ok && !mbar_wait(pv_done + ((g0 + num_kt - 1) & 1), ((g0 + num_kt - 1) >> 1) & 1, abort_word)) ok = false;
            if (!ok) break;
            tc_fence_after();
            if (splits > 1) {
                // the merge kernel divides: O as accumulated (scaled by 2^-m_ref), m_ref and the sum
                float* dst_o = part_o + part_slot * D;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_load32_nowait(lane_base + Cfg::O_COL + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<uint4*>(dst_o + c * 32 + i * 4) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                    }
                }
                if (valid) {
                    part_ml[part_slot * 2] = m_ref;
                    part_ml[part_slot * 2 + 1] = l;
                }
                tc_fence_before();
                g0 += num_kt;
                continue;
            }
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = out + (size_t)(t.tok0 + t.q0 + r) * out_stride + (size_t)h * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_load32_nowait(lane_base + Cfg::O_COL + c * 32, o);
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 2 * e]) * inv,
                                                                        __uint_as_float(o[8 * i + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<uint32_t*>(&pair);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            tc_fence_before();  // the reads of O are done before this thread's next arrival lets the next tile's P V overwrite it
            g0 += num_kt;
        }
        if (!ok) {
            if (lane == 0 && !*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
            *abort_word = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_word && threadIdx.x == 0) {
        // copies that are still in flight target this block's shared memory: one more short wait
        // on the barriers they complete (q_full, k_full, v_full), whichever phase they are in
        volatile int ignore = 0;
        for (int s = 0; s < 1 + 2 * FA_STAGES; ++s) {
            mbar_wait(bars + s, 0, &ignore, 1024);
            mbar_wait(bars + s, 1, &ignore, 1024);
        }
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLUMNS);
    }
}

// ------------------------------------------------------------------ two query tiles a block
// For long portions (head_dim 128): a block owns two consecutive tiles of 128 queries, A and B, of one
// head and walks the keys in tiles of 128.  Each K and V tile is copied once for both; S_A, S_B, O_A and
// O_B fill the SM's 512 columns of tensor memory (one block an SM), and each query tile has four softmax
// warps of its own.  The products of one tile run while the other's softmax works, in this order on the
// tensor pipe:  Q_A K_0, Q_B K_0, | P_A V_0, Q_A K_1, | P_B V_0, Q_B K_1, | P_A V_1, Q_A K_2, ...
// S_X has one buffer, which P_X overwrites: Q_X K_{i+1} is issued behind P_X V_i, so when the softmax
// sees S_X of a tile every product into O_X before it is complete (the tensor pipe keeps the order),
// and a rescale of O_X needs no barrier of its own.
#define FB_THREADS 384  // three warpgroups: roles (producer, products, two idle warps), softmax of tile A, softmax of tile B
#define FB_BN 128

struct FbCfg {  // head_dim 128
    static constexpr int D = 128;
    static constexpr int BANDS = 2;
    static constexpr int Q_BAND = FA_BM * 128;   // bytes of one 64-column band of a Q tile
    static constexpr int Q_BYTES = BANDS * Q_BAND;
    static constexpr int KV_BAND = FB_BN * 128;  // bytes of one band of a K tile
    static constexpr int KV_BYTES = BANDS * KV_BAND;
    static constexpr int STAGES = 2;
    static constexpr int OFF_K = 2 * Q_BYTES;
    static constexpr int OFF_V = OFF_K + STAGES * KV_BYTES;
    static constexpr int OFF_BAR = OFF_V + STAGES * KV_BYTES;
    static constexpr int NUM_BARS = 1 + 4 * STAGES + 2 + 2 + 2;
    static constexpr size_t SMEM = OFF_BAR + NUM_BARS * 8 + 16;
    static constexpr int S_COL = 0;    // S_A at 0, S_B at 128; P_X (bf16 pairs) overwrites the first 64 columns of S_X
    static constexpr int O_COL = 256;  // O_A at 256, O_B at 384
    static constexpr int TMEM_COLUMNS = 512;
};

// tile_rows / tile_starts list tiles of 256 queries here.
__global__ void __launch_bounds__(FB_THREADS, 1)
attention_prefill_tc5_two_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int out_stride,
                                 const int* __restrict__ qo_indptr, const int* __restrict__ seq_lens,
                                 const int* __restrict__ block_table, int max_pages, const int* __restrict__ tile_rows,
                                 const int* __restrict__ tile_starts, int num_tiles, int Hq, int Hkv, int page_size, int page_shift,
                                 int num_pages, float scale, int window, int merged, int* flag) {
    using Cfg = FbCfg;
    constexpr int D = Cfg::D;
    constexpr int BANDS = Cfg::BANDS;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* sQ = smem;
    unsigned char* sK = smem + Cfg::OFF_K;
    unsigned char* sV = smem + Cfg::OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = k_full + Cfg::STAGES;
    uint64_t* k_empty = v_full + Cfg::STAGES;
    uint64_t* v_empty = k_empty + Cfg::STAGES;
    uint64_t* s_full = v_empty + Cfg::STAGES;  // [A, B]
    uint64_t* p_full = s_full + 2;             // [A, B]
    uint64_t* o_done = p_full + 2;             // [A, B]: the last product into O_X is complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(k_full + s, 1);
            mbar_init(v_full + s, 1);
            mbar_init(k_empty + s, 1);
            mbar_init(v_empty + s, 1);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(s_full + x, 1);
            mbar_init(p_full + x, 4);
            mbar_init(o_done + x, 1);
        }
        *abort_word = 0;
        if ((smem_addr(smem) & 1023u) != 0) {
            if (flag) atomicOr(flag, KB_FLAG_MISALIGNED);
            *abort_word = 1;
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    const int h = blockIdx.x;
    const int kvh = h / (Hq / Hkv);
    const int tile = num_tiles - 1 - (int)blockIdx.y;  // the longest first
    const int row = tile_rows[tile];
    const int q0 = tile_starts[tile];
    const int tok0 = qo_indptr[row];
    const int chunk_len = qo_indptr[row + 1] - tok0;
    const int seq_len = seq_lens[row];
    const int chunk_pos = seq_len - chunk_len;
    // per query tile X: rows, positions, the key tiles (of 128) it may see (scalars, picked by X: no indexed arrays)
    struct Side {
        int rows, first_pos, last_pos, first_kt, last_kt;
    };
    auto side_of = [&](int x) {
        Side t;
        t.rows = max(0, min(FA_BM, chunk_len - q0 - x * FA_BM));
        t.first_pos = chunk_pos + q0 + x * FA_BM;
        t.last_pos = t.first_pos + max(t.rows, 1) - 1;
        const int key_lo = (window > 0 && t.first_pos + 1 > window) ? t.first_pos + 1 - window : 0;
        t.first_kt = key_lo / FB_BN;
        t.last_kt = t.rows > 0 ? t.last_pos / FB_BN : -1;  // without rows: no tile
        return t;
    };
    const Side side_a = side_of(0), side_b = side_of(1);
    const bool has_b = side_b.rows > 0;
    const int first = side_a.first_kt;
    const int last = has_b ? side_b.last_kt : side_a.last_kt;
    const int n = last - first + 1;
    const int key_end = (has_b ? side_b.last_pos : side_a.last_pos) + 1;  // keys from here on belong to nobody: never read as data
    auto active = [&](int x, int i) {
        const int lo_kt = x ? side_b.first_kt : side_a.first_kt;
        const int hi_kt = x ? side_b.last_kt : side_a.last_kt;
        return first + i >= lo_kt && first + i <= hi_kt;
    };

    const int box_rows = page_size < FA_BN ? page_size : FA_BN;  // rows of a copy (the cache maps' boxes hold at most 64)
    const int run_rows = merged ? box_rows : FB_BN;
    const int band_bytes = run_rows * 128;
    const int run_bytes = BANDS * band_bytes;

    // The softmax warps hold a row of 128 scores in registers: the role warpgroup gives up registers, the two
    // softmax warpgroups take them (168 a thread at launch: 72 / 208 / 208 after).
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    if (*abort_word || warp >= 2) {
        // fall through to the common exit
    } else if (warp == 0) {
        // ---------------- producer
        const int runs = FB_BN / box_rows;
        const int per_k = BANDS * runs;
        const int per_v = merged ? runs : BANDS * runs;
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, (has_b ? 2 : 1) * Cfg::Q_BYTES);
            for (int x = 0; x < (has_b ? 2 : 1); ++x)
#pragma unroll
                for (int band = 0; band < BANDS; ++band)
                    tma_load_2d_plain(sQ + x * Cfg::Q_BYTES + band * Cfg::Q_BAND, &map_q, h * D + band * 64, tok0 + q0 + x * FA_BM, q_full);
        }
        const int* table = block_table + (size_t)row * max_pages;
        bool ok = true;
        for (int i = 0; i < n && ok; ++i) {
            const int st = i % Cfg::STAGES;
            const int use = i / Cfg::STAGES;
#pragma unroll
            for (int is_v = 0; is_v < 2; ++is_v) {
                if (use > 0 && !mbar_wait((is_v ? v_empty : k_empty) + st, (use - 1) & 1, abort_word)) {
                    if (lane == 0 && !*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
                    *abort_word = 1;
                    ok = false;
                    break;
                }
                uint64_t* bar = (is_v ? v_full : k_full) + st;
                if (lane == 0) mbar_arrive_expect_tx(bar, Cfg::KV_BYTES);
                __syncwarp();
                for (int op = lane; op < (is_v ? per_v : per_k); op += 32) {
                    const int band = op / runs;
                    const int run = op % runs;
                    const int key = (first + i) * FB_BN + run * box_rows;
                    const int page_index = key >> page_shift;
                    int page = 0, within = 0;  // the reserved page stands in for rows nobody may see
                    if (key < key_end && page_index < max_pages) {
                        const int p = table[page_index];
                        if (p >= 0 && p < num_pages) {
                            page = p;
                            within = key - (page_index << page_shift);
                        }
                    }
                    unsigned char* tile_base = (is_v ? sV : sK) + st * Cfg::KV_BYTES;
                    if (is_v && merged)
                        tma_load_5d_plain(tile_base + run * run_bytes, &map_v, 0, kvh, within, 0, page, bar);
                    else
                        tma_load_4d_plain(tile_base + band * Cfg::KV_BAND + run * box_rows * 128, is_v ? &map_v : &map_k, band * 64, kvh, within, page, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc(FB_BN);
            constexpr uint32_t idesc_pv = umma_idesc_b_mn(D);
            const uint64_t q_desc = umma_desc_sw128(smem_addr(sQ));
            const uint64_t k_desc = umma_desc_sw128(smem_addr(sK));
            const uint64_t v_desc = umma_desc_mn_sw128(smem_addr(sV), (uint32_t)band_bytes, 1024);
            uint64_t v_step[FB_BN / 16];  // where the 16 keys of a P V step lie in a V tile (see the one-tile kernel)
#pragma unroll
            for (int ks = 0; ks < FB_BN / 16; ++ks) {
                const int key = ks * 16;
                v_step[ks] = (uint64_t)(((key / run_rows) * run_bytes + (key % run_rows) * 128) >> 4);
            }
            bool ok = true;
            auto give_up = [&]() {
                if (!*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
                *abort_word = 1;
                ok = false;
            };
            auto issue_qk = [&](int x, int i) {  // S_X = Q_X K_i^T
                const uint64_t k_tile = k_desc + (uint64_t)(((i % Cfg::STAGES) * Cfg::KV_BYTES) >> 4);
                const uint64_t q_tile = q_desc + (uint64_t)((x * Cfg::Q_BYTES) >> 4);
#pragma unroll
                for (int band = 0; band < BANDS; ++band)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + Cfg::S_COL + x * FB_BN, q_tile + (uint64_t)((band * Cfg::Q_BAND + k * 32) >> 4),
                                  k_tile + (uint64_t)((band * Cfg::KV_BAND + k * 32) >> 4), idesc_qk, (band > 0 || k > 0) ? 1u : 0u);
                umma_commit(s_full + x);
            };
            int done_pv[2] = {0, 0};  // products into O_X issued so far = phase of p_full[X] to wait for next
            auto issue_pv = [&](int x, int i) {  // O_X += P_X V_i
                if (!mbar_wait(p_full + x, done_pv[x] & 1, abort_word)) {
                    give_up();
                    return;
                }
                tc_fence_after();
                const uint64_t v_tile = v_desc + (uint64_t)(((i % Cfg::STAGES) * Cfg::KV_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < FB_BN / 16; ++ks)
                    umma_bf16_a_tmem(tmem_base + Cfg::O_COL + x * D, tmem_base + Cfg::S_COL + x * FB_BN + ks * 8, v_tile + v_step[ks],
                                     idesc_pv, (done_pv[x] > 0 || ks > 0) ? 1u : 0u);
                ++done_pv[x];
                if (!active(x, i + 1)) umma_commit(o_done + x);  // that was X's last tile
            };
            if (!mbar_wait(q_full, 0, abort_word) || !mbar_wait(k_full, 0, abort_word)) give_up();
            if (ok) {
                tc_fence_after();
                if (active(0, 0)) issue_qk(0, 0);
                if (active(1, 0)) issue_qk(1, 0);
                umma_commit(k_empty);
            }
            for (int i = 0; i < n && ok; ++i) {
                const int st = i % Cfg::STAGES;
                const bool more = i + 1 < n;
                if (!mbar_wait(v_full + st, (i / Cfg::STAGES) & 1, abort_word)) {
                    give_up();
                    break;
                }
                tc_fence_after();
                if (active(0, i)) issue_pv(0, i);
                if (!ok) break;
                if (more) {
                    if (!mbar_wait(k_full + (i + 1) % Cfg::STAGES, ((i + 1) / Cfg::STAGES) & 1, abort_word)) {
                        give_up();
                        break;
                    }
                    tc_fence_after();
                    if (active(0, i + 1)) issue_qk(0, i + 1);
                }
                if (active(1, i)) issue_pv(1, i);
                if (!ok) break;
                umma_commit(v_empty + st);
                if (more) {
                    if (active(1, i + 1)) issue_qk(1, i + 1);
                    umma_commit(k_empty + (i + 1) % Cfg::STAGES);
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;\n");
        if (!*abort_word) {
        // ---------------- softmax and epilogue: warps 4-7 own query tile A, warps 8-11 tile B; thread r owns row r
        const int x = warp >= 8 ? 1 : 0;
        const int quarter = warp & 3;  // the TMEM lanes this warp may touch
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_col = lane_base + Cfg::S_COL + x * FB_BN;
        const uint32_t o_col = lane_base + Cfg::O_COL + x * D;
        const int soft_tid = (warp - 4 - 4 * x) * 32 + lane;  // 0..127 within the group
        const float sl2 = scale * FA_LOG2E;
        bool ok = true;
        const Side mine = x ? side_b : side_a;
        if (mine.rows > 0) {
            const bool valid = r < mine.rows;
            const int pos = valid ? mine.first_pos + r : mine.last_pos;
            const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            const int lo_last = (window > 0 && mine.last_pos + 1 > window) ? mine.last_pos + 1 - window : 0;
            float m_ref = -INFINITY;
            float l = 0.0f;
            int seen = 0;
            for (int i = 0; i < n; ++i) {
                if (!active(x, i)) continue;
                const int key0 = (first + i) * FB_BN;
                if (!mbar_wait(s_full + x, seen & 1, abort_word)) { ok = false; break; }
                tc_fence_after();
                const bool edge = key0 + FB_BN - 1 > mine.first_pos || key0 < lo_last;  // the diagonal or the window's edge crosses this tile
                // the row's 128 raw scores, fetched at once (one wait for four loads: a load's latency is paid once a tile)
                uint32_t raw[FB_BN / 32][32];
#pragma unroll
                for (int part = 0; part < FB_BN / 32; ++part) tmem_load32_nowait(s_col + part * 32, raw[part]);
                tmem_wait_ld();
                if (edge) {
#pragma unroll
                    for (int c = 0; c < FB_BN; ++c) {
                        const int key = key0 + c;
                        if (!(key <= pos && key >= lo)) raw[c >> 5][c & 31] = 0xff800000u;  // -inf
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < FB_BN; c += 8) {
                    mx4[0] = max3(mx4[0], __uint_as_float(raw[c >> 5][c & 31]), __uint_as_float(raw[c >> 5][(c & 31) + 1]));
                    mx4[1] = max3(mx4[1], __uint_as_float(raw[c >> 5][(c & 31) + 2]), __uint_as_float(raw[c >> 5][(c & 31) + 3]));
                    mx4[2] = max3(mx4[2], __uint_as_float(raw[c >> 5][(c & 31) + 4]), __uint_as_float(raw[c >> 5][(c & 31) + 5]));
                    mx4[3] = max3(mx4[3], __uint_as_float(raw[c >> 5][(c & 31) + 6]), __uint_as_float(raw[c >> 5][(c & 31) + 7]));
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;  // -inf stays -inf
                float alpha = 1.0f;
                if (m_ref == -INFINITY) {
                    m_ref = mx;
                } else if (mx > m_ref + FA_RESCALE_STEP) {
                    alpha = exp2f(m_ref - mx);
                    m_ref = mx;
                }
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    // every product into O_X issued so far is complete: S_X of this tile was computed behind them
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t o[32];
                        tmem_load32_nowait(o_col + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        tmem_store32(o_col + c * 32, o);
                    }
                    tmem_wait_st();
                    l *= alpha;
                }
                // P = 2^(s * scale - m_ref) as bf16 pairs over the first half of S_X (all of which is in registers), and the row's sum
                const float neg_base = m_ref == -INFINITY ? 0.0f : -m_ref;
                const float2 scale2 = make_float2(sl2, sl2);
                const float2 base2 = make_float2(neg_base, neg_base);
                float2 sum2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t packed[32];
#pragma unroll
                    for (int c = 0; c < 64; c += 2) {
                        const int col = half * 64 + c;
                        const float2 arg = ffma2(make_float2(__uint_as_float(raw[col >> 5][col & 31]), __uint_as_float(raw[col >> 5][(col & 31) + 1])),
                                                 scale2, base2);  // (-inf) * scale + base = -inf
                        const float2 pr = make_float2(ex2_ftz(arg.x), ex2_ftz(arg.y));
                        sum2[(c >> 1) & 1] = fadd2(sum2[(c >> 1) & 1], pr);
                        __nv_bfloat162 pair = __floats2bfloat162_rn(pr.x, pr.y);
                        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    tmem_store32(s_col + half * 32, packed);
                }
                l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
                tmem_wait_st();
                if (key0 + FB_BN > key_end) {
                    // rows of V beyond the last query: P is 0 there, but 0 * NaN is NaN
                    const int st = i % Cfg::STAGES;
                    if (!mbar_wait(v_full + st, (i / Cfg::STAGES) & 1, abort_word)) { ok = false; break; }
                    unsigned char* v_tile = sV + st * Cfg::KV_BYTES;
                    for (int idx = soft_tid; idx < FB_BN * BANDS * 8; idx += 128) {
                        const int vr = idx / (BANDS * 8);
                        const int c = idx % (BANDS * 8);
                        if (key0 + vr >= key_end)
                            *reinterpret_cast<uint4*>(v_tile + (vr / run_rows) * run_bytes + (c >> 3) * band_bytes + (vr % run_rows) * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + x);
                ++seen;
            }
            if (ok && !mbar_wait(o_done + x, 0, abort_word)) ok = false;
            if (ok) {
                tc_fence_after();
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                __nv_bfloat16* dst = out + (size_t)(tok0 + q0 + x * FA_BM + r) * out_stride + (size_t)h * D;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_load32_nowait(o_col + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(o[8 * q + 2 * e]) * inv,
                                                                            __uint_as_float(o[8 * q + 2 * e + 1]) * inv);
                                w[e] = *reinterpret_cast<uint32_t*>(&pair);
                            }
                            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
                tc_fence_before();
            }
        }
        if (!ok) {
            if (lane == 0 && !*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT | KB_FLAG_TIMEOUT_PREFILL);
            *abort_word = 1;
        }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_word && threadIdx.x == 0) {
        volatile int ignore = 0;
        for (int s = 0; s < 1 + 2 * Cfg::STAGES; ++s) {
            mbar_wait(bars + s, 0, &ignore, 1024);
            mbar_wait(bars + s, 1, &ignore, 1024);
        }
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLUMNS);
    }
}

// Combines the splits of the keys: a warp per (query, head); lane i owns D / 32 columns.
// part_o: [splits, tiles * 128, Hq, D] as the blocks accumulated it, part_ml: the same slots x (reference
// maximum, sum).  out = sum_z 2^(m_z - M) O_z / sum_z 2^(m_z - M) l_z, in split order.
template <int D>
__global__ void attention_prefill_tc5_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                   const int* __restrict__ qo_indptr, const int* __restrict__ tile_rows,
                                                   const int* __restrict__ tile_starts, int num_tiles, int Hq, int splits,
                                                   __nv_bfloat16* __restrict__ out, int out_stride) {
    constexpr int PER = D / 32;
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (tile, row of the tile, head)
    const long long slots = (long long)num_tiles * FA_BM;
    if (pair >= slots * Hq) return;
    const int h = (int)(pair % Hq);
    const int slot = (int)(pair / Hq);
    const int tile = slot / FA_BM, r = slot % FA_BM;
    const int row = tile_rows[tile];
    const int tok0 = qo_indptr[row];
    const int q0 = tile_starts[tile];
    if (q0 + r >= qo_indptr[row + 1] - tok0) return;  // the tile's last rows lie beyond the portion
    pdl_wait();
    float big = -INFINITY;
    for (int z = 0; z < splits; ++z) big = fmaxf(big, part_ml[(((size_t)z * slots + slot) * Hq + h) * 2]);
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.0f;
    float den = 0.0f;
    for (int z = 0; z < splits; ++z) {
        const size_t at = ((size_t)z * slots + slot) * Hq + h;
        const float m = part_ml[at * 2];
        if (m == -INFINITY) continue;  // a split without keys this row may see: its O was not written or is all zero
        const float f = exp2f(m - big);
        den += part_ml[at * 2 + 1] * f;
        float part[PER];
        if (PER == 4)
            *reinterpret_cast<float4*>(part) = *reinterpret_cast<const float4*>(part_o + at * D + lane * PER);
        else
            *reinterpret_cast<float2*>(part) = *reinterpret_cast<const float2*>(part_o + at * D + lane * PER);
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += part[i] * f;
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    __nv_bfloat16* dst = out + (size_t)(tok0 + q0 + r) * out_stride + (size_t)h * D + lane * PER;
    uint32_t packed[PER / 2];
#pragma unroll
    for (int i = 0; i < PER; i += 2) {
        __nv_bfloat162 two = __floats2bfloat162_rn(acc[i] * inv, acc[i + 1] * inv);
        packed[i / 2] = *reinterpret_cast<uint32_t*>(&two);
    }
    if (PER == 4)
        *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[PER / 2 - 1]);
    else
        *reinterpret_cast<uint32_t*>(dst) = packed[0];
}

static int fa_resident(int blocks_per_sm) {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 148;
    }
    return sms * blocks_per_sm;
}

// Blocks that share a query tile's keys: more than one when a step's tiles (a short portion of a
// long prompt: 4 tiles x 32 heads) would leave most of the device idle.  Every split gets at least
// four key tiles of the longest row; at most eight splits.
KB_EXPORT int kb_attention_prefill_tc5_splits(int D, int Hq, int num_tiles, int max_seq_len) {
    if (D != 64 && D != 128) return 1;
    const long long blocks = (long long)Hq * num_tiles;
    if (blocks < 1) return 1;
    const int resident = fa_resident(FaCfg<128>::BLOCKS_PER_SM);
    long long splits = resident / blocks;
    const int key_tiles = (max_seq_len + FA_BN - 1) / FA_BN;
    if (splits > key_tiles / 4) splits = key_tiles / 4;
    if (splits > 8) splits = 8;
    return splits < 2 ? 1 : (int)splits;
}

template <int D>
static int launch_fa(const CUtensorMap* mq, const CUtensorMap* mk, const CUtensorMap* mv, __nv_bfloat16* out, int out_stride,
                     const int* qo_indptr, const int* seq_lens, const int* block_table, int max_pages, const int* tile_rows,
                     const int* tile_starts, int num_tiles, int Hq, int Hkv, int page_size, int num_pages, float scale, int window,
                     int merged, int splits, float* part_o, float* part_ml, int* flag, cudaStream_t stream) {
    const size_t smem = FaCfg<D>::SMEM;
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc5_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;  // page_size is a power of two here
    // Two tiles a block (one from each end of the list) when one tile a block would not run all at
    // once but two tiles a block do; with the keys split over blocks, one tile a block.
    const int resident = fa_resident(FaCfg<D>::BLOCKS_PER_SM);
    const long long single = (long long)Hq * num_tiles;
    const int paired = splits == 1 && num_tiles > 1 && single > resident && (long long)Hq * ((num_tiles + 1) / 2) <= resident ? 1 : 0;
    dim3 grid(Hq, paired ? (num_tiles + 1) / 2 : num_tiles, splits);
    kb_launch(attention_prefill_tc5_kernel<D>, dim3(grid), dim3(FA_THREADS), smem, stream, *mq, *mk, *mv, out, out_stride, qo_indptr,
              seq_lens, block_table, max_pages, tile_rows, tile_starts, num_tiles, Hq, Hkv, page_size, shift, num_pages, scale, window, merged,
              paired, splits, part_o, part_ml, flag);
    int rc = kb_launch_result();
    if (rc != 0 || splits == 1) return rc;
    const long long pairs = (long long)num_tiles * FA_BM * Hq;
    kb_launch(attention_prefill_tc5_merge_kernel<D>, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, stream, (const float*)part_o,
              (const float*)part_ml, qo_indptr, tile_rows, tile_starts, num_tiles, Hq, splits, out, out_stride);
    return kb_launch_result();
}

static int launch_two(const CUtensorMap* mq, const CUtensorMap* mk, const CUtensorMap* mv, __nv_bfloat16* out, int out_stride,
                      const int* qo_indptr, const int* seq_lens, const int* block_table, int max_pages, const int* wide_rows,
                      const int* wide_starts, int num_wide, int Hq, int Hkv, int page_size, int num_pages, float scale, int window,
                      int merged, int* flag, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc5_two_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FbCfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    dim3 grid(Hq, num_wide);
    kb_launch(attention_prefill_tc5_two_kernel, dim3(grid), dim3(FB_THREADS), FbCfg::SMEM, stream, *mq, *mk, *mv, out, out_stride, qo_indptr,
              seq_lens, block_table, max_pages, wide_rows, wide_starts, num_wide, Hq, Hkv, page_size, shift, num_pages, scale, window, merged,
              flag);
    return kb_launch_result();
}

// Whether a step's portions go to the kernel that takes two query tiles a block (head_dim 128,
// lists of 256-query tiles given): when its blocks, one an SM, make two waves or more, or one wave
// over long rows.  Measured on 32 heads, pages of 16 (us a layer, one tile a block / two):
// 2,048 tokens 55.5 / 57.0; 4,096: 177 / 169; 8,192: 596 / 555; 2,048 tokens at the end of 8,192:
// 318 / 273; 16,384: 2,250 / 2,242.  With pages of 64 positions the one-tile kernel needs few copies
// and stays ahead (8,192 tokens: 529 / 555).
KB_EXPORT int kb_attention_prefill_tc5_two_tiles(int D, int Hq, int num_wide, int page_size, int max_seq_len) {
    if (D != 128 || num_wide < 1 || page_size >= 64) return 0;
    const long long blocks = (long long)Hq * num_wide;
    const long long wave = fa_resident(1);
    return (blocks >= 2 * wave || (blocks >= wave && max_seq_len >= 4096)) ? 1 : 0;
}

// 1 when (head_dim, page_size) fit this kernel.
KB_EXPORT int kb_attention_prefill_tc5_supported(int D, int page_size) {
    if (D != 64 && D != 128) return 0;
    if (page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
    return 1;
}

// 1 when the kernel wants a map of V whose boxes take every 64-column band at once
// (kb_attention_encode_cache_map with bands = 1) for this head_dim and page size.
KB_EXPORT int kb_attention_prefill_tc5_merged(int D, int page_size) { return D > 64 && page_size >= 16 ? 1 : 0; }

// map_q: 2-D map over the packed qkv rows [tokens, q_stride] with boxes of [128 rows, 64 columns];
// map_k, map_v: maps over the caches [pages, page_size, kv_heads, head_dim]: 4-D with boxes of
// 64 columns x 1 head x min(page_size, 64) positions x 1 page; map_v, where
// kb_attention_prefill_tc5_merged says so, 5-D with every band in a box; all with the 128-byte
// swizzle (host pointers).  The tile list holds 128 queries per tile.  splits (1, or what
// kb_attention_prefill_tc5_splits gives): blocks that share a tile's keys; with more than one,
// part_o [splits, tiles * 128, Hq, D] and part_ml [splits, tiles * 128, Hq, 2] floats hold their results
// until a second kernel combines them.  two_tiles (what kb_attention_prefill_tc5_two_tiles gives, or 0): the
// portions go to the kernel that takes two query tiles a block, whose list (wide_rows, wide_starts,
// num_wide) holds 256 queries per tile.
KB_EXPORT int kb_attention_prefill_tc5(const void* map_q, const void* map_k, const void* map_v, void* out, int out_stride,
                                       const int* qo_indptr, const int* seq_lens, const int* block_table, int max_pages,
                                       const int* tile_rows, const int* tile_starts, int num_tiles, int Hq, int Hkv, int D,
                                       int page_size, int num_pages, float scale, int window, int splits, float* part_o,
                                       float* part_ml, const int* wide_rows, const int* wide_starts, int num_wide, int two_tiles,
                                       int* flag, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if (two_tiles && (D != 128 || splits != 1 || !wide_rows || !wide_starts || num_wide < 1 || num_wide > 65535)) return KB_ERR_BAD_ARG;
    if (splits < 1 || splits > 8 || (splits > 1 && (!part_o || !part_ml || ((uintptr_t)part_o % 16) != 0))) return KB_ERR_BAD_ARG;
    if (!map_q || !map_k || !map_v || !out || !qo_indptr || !seq_lens || !block_table || !tile_rows || !tile_starts) return KB_ERR_NULL;
    if (Hkv < 1 || Hq % Hkv != 0 || num_tiles > 65535) return KB_ERR_BAD_ARG;
    if (out_stride % 8 != 0 || ((uintptr_t)out % 16) != 0) return KB_ERR_BAD_ARG;  // 16-byte stores of whole rows
    if (!kb_attention_prefill_tc5_supported(D, page_size)) return KB_ERR_UNSUPPORTED_SIZE;
#define ARGS (const CUtensorMap*)map_q, (const CUtensorMap*)map_k, (const CUtensorMap*)map_v, (__nv_bfloat16*)out, out_stride, qo_indptr, \
             seq_lens, block_table, max_pages, tile_rows, tile_starts, num_tiles, Hq, Hkv, page_size, num_pages, scale, window,            \
             kb_attention_prefill_tc5_merged(D, page_size), splits, part_o, part_ml, flag, stream
    if (two_tiles)
        return launch_two((const CUtensorMap*)map_q, (const CUtensorMap*)map_k, (const CUtensorMap*)map_v, (__nv_bfloat16*)out, out_stride,
                          qo_indptr, seq_lens, block_table, max_pages, wide_rows, wide_starts, num_wide, Hq, Hkv, page_size, num_pages, scale,
                          window, kb_attention_prefill_tc5_merged(D, page_size), flag, stream);
    if (D == 64) return launch_fa<64>(ARGS);
    return launch_fa<128>(ARGS);
#undef ARGS
}
