// Weight-streaming matrix product on the 5th-generation tensor cores:
//     out[M, N] = x[M, K] . W[N, K]^T (+ bias),   M <= 64 tokens, bf16 in, fp32 accumulate,
// optionally gated:  out[M, N/2] = silu(x.Wg^T) * (x.Wu^T), Wg = W[:N/2], Wu = W[N/2:]
// (kairyu/models/layers.py:244).
//
// The roles are swapped with respect to the usual product: 128 rows of W are the M side of
// tcgen05.mma, the (padded) tokens its N side, so that a block streams a 128-row band of W
// exactly once.  One thread feeds the pipeline with TMA (cp.async.bulk.tensor, 128-byte
// swizzle, W with an evict-first and x with an evict-last L2 hint), one thread issues
// tcgen05.mma into a TMEM accumulator, four warps read the accumulator back with tcgen05.ld
// and write the result.  Small N is covered by splitting K over blocks; their fp32 partial
// sums are added in split order by a second kernel, so the result does not depend on timing.
//
// Every wait on an mbarrier is bounded: a block that gives up raises KB_FLAG_TIMEOUT, lets
// its other roles leave through a shared abort word, frees its TMEM and returns.
#include "umma.cuh"

#define TC_THREADS 192
#define TC_BLOCK_K 64      // k per pipeline stage: 128 bytes of bf16, one swizzle row
#define TC_SMEM_BUDGET (200 * 1024)

template <int NTOK, bool GATED>
struct TcConfig {
    static constexpr int BANDS = GATED ? 2 : 1;
    static constexpr int A_BYTES = TC_BLOCK_ROWS * TC_BLOCK_K * 2;  // one band of W per stage
    static constexpr int B_BYTES = NTOK * TC_BLOCK_K * 2;
    static constexpr int STAGE_BYTES = BANDS * A_BYTES + B_BYTES;
    static constexpr int STAGES = TC_SMEM_BUDGET / STAGE_BYTES;
    static constexpr int TMEM_COLUMNS = (BANDS * NTOK) <= 32 ? 32 : ((BANDS * NTOK) <= 64 ? 64 : ((BANDS * NTOK) <= 128 ? 128 : 256));
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + (2 * STAGES + 1) * 8 + 16;
};

// grid (ceil(rows_out / 128), k_splits).  partial != null: fp32 partial sums
// [k_splits, M, N_out] are written instead of out (bias and gate are not applied).
template <int NTOK, bool GATED>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, void* __restrict__ out,
                int out_fp32, int ldo, const __nv_bfloat16* __restrict__ bias, float* __restrict__ partial, int M, int N, int K,
                int k_blocks_per_split, int rows_per_block, int* flag) {
    using Cfg = TcConfig<NTOK, GATED>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_base = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + Cfg::STAGES;
    uint64_t* done_bar = empty_bar + Cfg::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rows_out = GATED ? N / 2 : N;
    // A block owns rows_per_block (<= 128) weight rows: the copies bring only those (the box of map_w
    // is that high), the other rows of the 128-row MMA tile hold whatever the shared memory held and
    // their TMEM lanes are never read.  Fewer than 128 lets the host spread the rows over every SM.
    const int n0 = blockIdx.x * rows_per_block;
    const uint32_t stage_tx = (uint32_t)(Cfg::BANDS * rows_per_block * TC_BLOCK_K * 2 + Cfg::B_BYTES);
    const int total_k_blocks = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;
    const int kb_begin = blockIdx.y * k_blocks_per_split;
    const int kb_end = min(kb_begin + k_blocks_per_split, total_k_blocks);
    const int num_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 1);
        }
        mbar_init(done_bar, 1);
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLUMNS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------- producer: TMA loads of the W band(s) and the token tile
        const uint64_t stream_policy = policy_evict_first();
        const uint64_t keep_policy = policy_evict_last();
        // The weights do not depend on the kernel before this one: the first round of W
        // tiles is requested before the wait, the token tiles (that kernel's output) after.
        const int first_round = min(num_kb, (int)Cfg::STAGES);
        for (int i = 0; i < first_round; ++i) {
            unsigned char* a = stage_base + (size_t)i * Cfg::STAGE_BYTES;
            const int k = (kb_begin + i) * TC_BLOCK_K;
            mbar_arrive_expect_tx(full_bar + i, stage_tx);
            tma_load_2d(a, &map_w, k, n0, full_bar + i, stream_policy);
            if (GATED) tma_load_2d(a + Cfg::A_BYTES, &map_w, k, rows_out + n0, full_bar + i, stream_policy);
        }
        pdl_wait();
        for (int i = 0; i < first_round; ++i) {
            unsigned char* b = stage_base + (size_t)i * Cfg::STAGE_BYTES + Cfg::BANDS * Cfg::A_BYTES;
            tma_load_2d(b, &map_x, (kb_begin + i) * TC_BLOCK_K, 0, full_bar + i, keep_policy);
        }
        for (int i = first_round; i < num_kb; ++i) {
            const int s = i % Cfg::STAGES;
            const uint32_t round = i / Cfg::STAGES;
            if (!mbar_wait(empty_bar + s, (round & 1) ^ 1, abort_word)) {
                if (!*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT);
                *abort_word = 1;
                break;
            }
            unsigned char* a = stage_base + (size_t)s * Cfg::STAGE_BYTES;
            unsigned char* b = a + Cfg::BANDS * Cfg::A_BYTES;
            const int k = (kb_begin + i) * TC_BLOCK_K;
            mbar_arrive_expect_tx(full_bar + s, stage_tx);
            tma_load_2d(a, &map_w, k, n0, full_bar + s, stream_policy);
            if (GATED) tma_load_2d(a + Cfg::A_BYTES, &map_w, k, rows_out + n0, full_bar + s, stream_policy);
            tma_load_2d(b, &map_x, k, 0, full_bar + s, keep_policy);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc = umma_idesc(NTOK);
        bool ok = true;
        for (int i = 0; i < num_kb && ok; ++i) {
            const int s = i % Cfg::STAGES;
            const uint32_t round = i / Cfg::STAGES;
            if (!mbar_wait(full_bar + s, round & 1, abort_word)) {
                if (!*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT);
                *abort_word = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t a = smem_addr(stage_base + (size_t)s * Cfg::STAGE_BYTES);
            const uint32_t b = a + Cfg::BANDS * Cfg::A_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BLOCK_K / 16; ++k) {  // 16 k = 32 bytes along the swizzled row
                const uint64_t b_desc = umma_desc_sw128(b + k * 32);
                umma_bf16(tmem_base, umma_desc_sw128(a + k * 32), b_desc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                if (GATED) umma_bf16(tmem_base + NTOK, umma_desc_sw128(a + Cfg::A_BYTES + k * 32), b_desc, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar + s);  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(done_bar);    // the accumulator is complete
    } else if (warp >= 2) {
        // ---------------- epilogue: TMEM -> registers -> global
        pdl_wait();  // the output (or the partial-sum scratch) may still be read by the kernel before
        const bool ready = num_kb > 0 && mbar_wait(done_bar, 0, abort_word);
        if (!ready && num_kb > 0) {
            if (lane == 0 && !*abort_word && flag) atomicOr(flag, KB_FLAG_TIMEOUT);
            *abort_word = 1;
        }
        if (ready) {
            tc_fence_after();
            const int quarter = warp & 3;  // the TMEM lanes a warp may read
            const int row = quarter * 32 + lane;
            const int n = n0 + row;
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int c = 0; c < NTOK / 16; ++c) {
                float v[16], u[16];
                tmem_load16(lane_base + c * 16, v);
                if (GATED) tmem_load16(lane_base + NTOK + c * 16, u);
                if (row < rows_per_block && n < rows_out) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int token = c * 16 + j;
                        if (token >= M) break;
                        float value = v[j];
                        if (partial != nullptr) {
                            partial[((size_t)blockIdx.y * M + token) * rows_out + n] = value;
                            continue;
                        }
                        if (GATED) {
                            float up = u[j];
                            if (bias) {
                                value += __bfloat162float(bias[n]);
                                up += __bfloat162float(bias[rows_out + n]);
                            }
                            value = value / (1.0f + expf(-value)) * up;
                        } else if (bias) {
                            value += __bfloat162float(bias[n]);
                        }
                        if (out_fp32)
                            reinterpret_cast<float*>(out)[(size_t)token * ldo + n] = value;
                        else
                            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)token * ldo + n] = __float2bfloat16_rn(value);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLUMNS);
    }
}

// out[t, n] = sum_s partial[s, t, n] (+ bias[n]) in split order.
template <typename TO>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, const __nv_bfloat16* __restrict__ bias, TO* __restrict__ out,
                                     int ldo, int M, int N, int splits) {
    pdl_wait();
    const size_t total = (size_t)M * N;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / N);
        const int n = (int)(idx % N);
        float sum = 0.0f;
        for (int s = 0; s < splits; ++s) sum += partial[(size_t)s * total + idx];
        if (bias) sum += __bfloat162float(bias[n]);
        out[(size_t)t * ldo + n] = from_float<TO>(sum);
    }
}

// ------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled g_encode = nullptr;

static int get_encoder() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
    if (e != cudaSuccess) return (int)e;
    if (status != cudaDriverEntryPointSuccess || fn == nullptr) return KB_ERR_UNSUPPORTED_SIZE;
    g_encode = (PFN_cuTensorMapEncodeTiled)fn;
    return 0;
}

// Writes a 128-byte tensor map (host memory, 64-byte aligned) for a row-major bf16 matrix
// [rows, cols] with `row_stride` elements between rows; boxes are [box_rows, 64] elements with
// the 128-byte swizzle; out-of-range elements read as zero.
KB_EXPORT int kb_tc5_encode_map(void* map_out, const void* base, long long rows, long long cols, long long row_stride,
                                int box_rows) {
    if (!map_out || !base) return KB_ERR_NULL;
    if (((uintptr_t)map_out % 64) != 0 || ((uintptr_t)base % 16) != 0) return KB_ERR_BAD_ARG;
    if (rows < 1 || cols < 1 || (row_stride * 2) % 16 != 0 || box_rows < 1 || box_rows > 256) return KB_ERR_UNSUPPORTED_SIZE;
    const int rc = get_encoder();
    if (rc != 0) return rc;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    cuuint32_t box[2] = {TC_BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int NTOK, bool GATED>
static int launch_tc5(const CUtensorMap* map_w, const CUtensorMap* map_x, void* out, int out_fp32, int ldo,
                      const __nv_bfloat16* bias, float* partial, int M, int N, int K, int k_splits, int rows_per_block, int* flag,
                      cudaStream_t stream) {
    using Cfg = TcConfig<NTOK, GATED>;
    static_assert(Cfg::STAGES >= 2, "pipeline needs two stages");
    cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<NTOK, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    const int rows_out = GATED ? N / 2 : N;
    const int total_kb = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;
    const int per_split = (total_kb + k_splits - 1) / k_splits;
    const int splits = (total_kb + per_split - 1) / per_split;  // every split has work
    dim3 grid((rows_out + rows_per_block - 1) / rows_per_block, splits);
    kb_launch(gemm_tc5_kernel<NTOK, GATED>, dim3(grid), dim3(TC_THREADS), Cfg::SMEM, stream, *map_w, *map_x, out, out_fp32, ldo, bias,
                                                                         splits > 1 ? partial : nullptr, M, N, K, per_split, rows_per_block, flag);
    int rc = kb_launch_result();
    if (rc != 0 || splits == 1) return rc;
    const size_t total = (size_t)M * rows_out;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    if (out_fp32)
        kb_launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, partial, bias, (float*)out, ldo, M, rows_out, splits);
    else
        kb_launch(splitk_reduce_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, partial, bias, (__nv_bfloat16*)out, ldo, M, rows_out, splits);
    return kb_launch_result();
}

// Splits of K this entry point will use for (N rows of output, K): the caller sizes
// `partial` as splits * M * N_out floats.
KB_EXPORT int kb_gemm_tc5_splits(int n_out, int K, int gated) {
    const int tiles = (n_out + TC_BLOCK_ROWS - 1) / TC_BLOCK_ROWS;
    const int total_kb = (K + TC_BLOCK_K - 1) / TC_BLOCK_K;
    if (gated || tiles >= 120) return 1;
    int splits = 148 / tiles;  // one block per SM at most: a second wave would double the time
    if (splits < 1) splits = 1;
    if (splits > 8) splits = 8;
    while (splits > 1 && total_kb / splits < 8) --splits;  // at least 8 k-blocks a split
    const int per_split = (total_kb + splits - 1) / splits;
    return (total_kb + per_split - 1) / per_split;
}

// Weight rows a block should own for (rows of output, K): a multiple of 8 up to 128.  Without a
// split of K the rows are spread over as many whole waves of one block per SM as it takes
// (14,336 rows: 104 a block, 138 blocks; 25,600 rows: 88 a block, 291 blocks = two waves).
KB_EXPORT int kb_gemm_tc5_rows(int n_out, int K, int gated) {
    if (kb_gemm_tc5_splits(n_out, K, gated) > 1) return TC_BLOCK_ROWS;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 148;
    for (int waves = 1; waves <= 64; ++waves) {
        int rows = (n_out + sms * waves - 1) / (sms * waves);
        rows = (rows + 7) / 8 * 8;
        if (rows <= TC_BLOCK_ROWS) return rows < 8 ? 8 : rows;
    }
    return TC_BLOCK_ROWS;
}

// map_w, map_x: host pointers to tensor maps made by kb_tc5_encode_map (W with box_rows =
// rows_per_block, as kb_gemm_tc5_rows gives it; x with box_rows = the padded token count 16, 32
// or 64).  Returns 0, a negative KB_ERR_* code or a positive cudaError_t.
KB_EXPORT int kb_gemm_tc5(const void* map_w, const void* map_x, void* out, int out_fp32, int ldo, const void* bias,
                          float* partial, int M, int N, int K, int gated, int rows_per_block, int* flag, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (!map_w || !map_x || !out) return KB_ERR_NULL;
    if (M < 1 || M > 64 || K < 8 || K % 8 != 0) return KB_ERR_UNSUPPORTED_SIZE;
    if (gated && N % 2 != 0) return KB_ERR_BAD_ARG;
    if (rows_per_block < 8 || rows_per_block > TC_BLOCK_ROWS || rows_per_block % 8 != 0) return KB_ERR_BAD_ARG;
    const int n_out = gated ? N / 2 : N;
    const int splits = kb_gemm_tc5_splits(n_out, K, gated);
    if (splits > 1 && partial == nullptr) return KB_ERR_NULL;
    const CUtensorMap* mw = (const CUtensorMap*)map_w;
    const CUtensorMap* mx = (const CUtensorMap*)map_x;
    const __nv_bfloat16* b = (const __nv_bfloat16*)bias;
#define GO(NT, G) return launch_tc5<NT, G>(mw, mx, out, out_fp32, ldo, b, partial, M, N, K, splits, rows_per_block, flag, stream)
    if (M <= 16) { if (gated) GO(16, true); else GO(16, false); }
    if (M <= 32) { if (gated) GO(32, true); else GO(32, false); }
    if (gated) GO(64, true); else GO(64, false);
#undef GO
}
