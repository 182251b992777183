// Token selection on the device: argmax, logit edits (penalties and masks),
// and temperature / min-p / top-k / top-p sampling with a stateless Gumbel-max
// draw (kairyu/engine/core/sampler.py:1198-1389, kairyu/kernels/sampling_gpu.py:51-128).
//
// Every reduction has a fixed order (over threads, warps, the blocks of a cluster, the chunks of
// a row), so a draw is a pure function of (logits row, parameters, seed): the same on every run
// and in every batch composition.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

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

// ------------------------------------------------------------------ log-probability report
// For report r over row rows[r] of the logits: the log-softmax value of one token, and the k
// largest log-softmax values with their indices, largest first, ties by the lower index
// (kairyu/engine/core/sampler.py:1423-1437: taken from the raw logits, before any edit or
// temperature).  values[r, 0] is the token's, values[r, 1 + i] and indices[r, i] the i-th largest.
//
// Two launches.  The first cuts a row into chunks (32 of them, or more for a vocabulary beyond
// 262,144) with a block each: the chunk's part of the log-sum-exp (running maximum, sum) and its own
// k best entries, found by k passes over the chunk, which the L1 holds after the first.  Pass i finds
// the best entry that comes after pass i-1's in the order (value down, index up), so nothing has to
// be remembered but the last.  The second launch, a block a report, adds the chunks' sums in chunk
// order and finds the k best among the chunks' candidates the same way.  (One block a row, k + 1
// passes over the whole row, took 250 us at 128,256 entries and k = 5.)
constexpr int REPORT_THREADS = 256;
constexpr int REPORT_WARPS = REPORT_THREADS / 32;
constexpr int REPORT_CHUNKS = 32;
constexpr int REPORT_MAX_CHUNK = 8192;
constexpr int REPORT_ABSENT = 0x7fffffff;

__host__ __device__ inline int report_chunk_len(int V) {
    int len = (V + REPORT_CHUNKS - 1) / REPORT_CHUNKS;
    if (len > REPORT_MAX_CHUNK) len = REPORT_MAX_CHUNK;
    return len < 1 ? 1 : len;
}
// scratch of (report, chunk): maximum, sum, then k (value, index) pairs
__host__ __device__ inline size_t report_scratch_floats(int k) { return 2 + 2 * (size_t)k; }

// whether (v, i) comes before (bv, bi) in the order: value down, index up; an absent entry comes last
__device__ __forceinline__ bool report_before(float v, int i, float bv, int bi) {
    return i != REPORT_ABSENT && (bi == REPORT_ABSENT || v > bv || (v == bv && i < bi));
}

// The block's first entry in the order, for every thread.  red_v / red_i: REPORT_WARPS entries.
__device__ void report_block_best(float& best, int& best_i, float* red_v, int* red_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (report_before(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    __syncthreads();  // the call before has been read
    if ((threadIdx.x & 31) == 0) { red_v[threadIdx.x >> 5] = best; red_i[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    best = red_v[0];
    best_i = red_i[0];
#pragma unroll
    for (int w = 1; w < REPORT_WARPS; ++w)
        if (report_before(red_v[w], red_i[w], best, best_i)) { best = red_v[w]; best_i = red_i[w]; }
}

// grid (reports, chunks)
__global__ void __launch_bounds__(REPORT_THREADS)
logprob_chunk_kernel(const float* __restrict__ logits, int ld, int V, const int* __restrict__ rows, int k, int chunk_len,
                     float* __restrict__ scratch) {
    pdl_wait();
    __shared__ float red_m[REPORT_WARPS];
    __shared__ float red_s[REPORT_WARPS];
    __shared__ int red_i[REPORT_WARPS];
    const int r = blockIdx.x;
    const int chunk = blockIdx.y;
    const float* x = logits + (size_t)rows[r] * ld;
    const int begin = chunk * chunk_len;
    const int end = min(V, begin + chunk_len);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* mine = scratch + ((size_t)r * gridDim.y + chunk) * report_scratch_floats(k);

    // the chunk's part of the log of the sum of exponentials, with the running maximum taken out
    float m = -INFINITY, sum = 0.0f;
    for (int i = begin + threadIdx.x; i < end; i += REPORT_THREADS) {
        const float v = x[i];
        if (v > m) {
            sum = sum * expf(m - v) + 1.0f;  // m = -inf: sum is 0 and stays finite
            m = v;
        } else if (v > -INFINITY) {
            sum += expf(v - m);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const float os = __shfl_xor_sync(0xffffffffu, sum, o);
        const float nm = fmaxf(m, om);
        if (nm > -INFINITY) sum = sum * expf(m - nm) + os * expf(om - nm);
        m = nm;
    }
    if (lane == 0) { red_m[warp] = m; red_s[warp] = sum; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float bm = red_m[0], bs = red_s[0];
        for (int w = 1; w < REPORT_WARPS; ++w) {
            const float nm = fmaxf(bm, red_m[w]);
            if (nm > -INFINITY) bs = bs * expf(bm - nm) + red_s[w] * expf(red_m[w] - nm);
            bm = nm;
        }
        mine[0] = bm;
        mine[1] = bs;
    }

    float prev_v = INFINITY;
    int prev_i = -1;
    for (int pass = 0; pass < k; ++pass) {
        float best = -INFINITY;
        int best_i = REPORT_ABSENT;
        if (prev_i != REPORT_ABSENT)  // else nothing is left: later passes find nothing either
            for (int i = begin + threadIdx.x; i < end; i += REPORT_THREADS) {
                const float v = x[i];
                const bool after = v < prev_v || (v == prev_v && i > prev_i);
                if (after && report_before(v, i, best, best_i)) { best = v; best_i = i; }
            }
        report_block_best(best, best_i, red_m, red_i);
        if (threadIdx.x == 0) {
            mine[2 + 2 * pass] = best;
            mine[2 + 2 * pass + 1] = __int_as_float(best_i);
        }
        prev_v = best;
        prev_i = best_i;
    }
}

// grid (reports)
__global__ void __launch_bounds__(REPORT_THREADS)
logprob_merge_kernel(const float* __restrict__ logits, int ld, int V, const int* __restrict__ rows, const int* __restrict__ tokens,
                     int tokens_by_row, int k, int chunks, const float* __restrict__ scratch, float* __restrict__ values,
                     int* __restrict__ indices) {
    pdl_wait();
    __shared__ float red_v[REPORT_WARPS];
    __shared__ int red_i[REPORT_WARPS];
    __shared__ float bcast;
    const int r = blockIdx.x;
    const int row = rows[r];
    const float* x = logits + (size_t)row * ld;
    const size_t per = report_scratch_floats(k);
    const float* mine = scratch + (size_t)r * chunks * per;
    if (threadIdx.x == 0) {
        float bm = mine[0], bs = mine[1];
        for (int c = 1; c < chunks; ++c) {  // in chunk order
            const float cm = mine[c * per], cs = mine[c * per + 1];
            const float nm = fmaxf(bm, cm);
            if (nm > -INFINITY) bs = bs * expf(bm - nm) + cs * expf(cm - nm);
            bm = nm;
        }
        const float lse = bm + logf(bs);
        bcast = lse;
        int token = tokens[tokens_by_row ? row : r];
        token = min(max(token, 0), V - 1);
        values[(size_t)r * (k + 1)] = x[token] - lse;
    }
    __syncthreads();
    const float lse = bcast;

    const int candidates = chunks * k;
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int pass = 0; pass < k; ++pass) {
        float best = -INFINITY;
        int best_i = REPORT_ABSENT;
        if (prev_i != REPORT_ABSENT)
            for (int j = threadIdx.x; j < candidates; j += REPORT_THREADS) {
                const float* entry = mine + (size_t)(j / k) * per + 2 + 2 * (j % k);
                const float v = entry[0];
                const int i = __float_as_int(entry[1]);
                if (i == REPORT_ABSENT) continue;
                const bool after = v < prev_v || (v == prev_v && i > prev_i);
                if (after && report_before(v, i, best, best_i)) { best = v; best_i = i; }
            }
        report_block_best(best, best_i, red_v, red_i);
        if (threadIdx.x == 0) {
            // fewer than k entries (k > V): the rest are marked absent
            values[(size_t)r * (k + 1) + 1 + pass] = best_i == REPORT_ABSENT ? -INFINITY : best - lse;
            indices[(size_t)r * k + pass] = best_i == REPORT_ABSENT ? -1 : best_i;
        }
        prev_v = best;
        prev_i = best_i;
    }
}

// Floats of scratch kb_logprob_report needs for this many reports of k entries over a vocabulary of V.
KB_EXPORT long long kb_logprob_report_scratch_floats(int reports, int V, int k) {
    if (reports < 1 || V < 1 || k < 0) return 0;
    const int len = report_chunk_len(V);
    const int chunks = (V + len - 1) / len;
    return (long long)reports * chunks * (long long)report_scratch_floats(k);
}

// values: [reports, k + 1] floats, indices: [reports, k] ints (k may be 0: the token's value only).
// tokens_by_row: the token of report r is tokens[rows[r]] (a step's sampled ids), else tokens[r].
// scratch: kb_logprob_report_scratch_floats(reports, V, k) floats.
KB_EXPORT int kb_logprob_report(const float* logits, int ld, int n_rows, int V, const int* rows, const int* tokens,
                                int tokens_by_row, int reports, int k, float* values, int* indices, float* scratch,
                                cudaStream_t stream) {
    if (reports == 0) return 0;
    if (!logits || !rows || !tokens || !values || !scratch || (k > 0 && !indices)) return KB_ERR_NULL;
    if (V < 1 || k < 0 || n_rows < 1) return KB_ERR_BAD_ARG;
    const int len = report_chunk_len(V);
    const int chunks = (V + len - 1) / len;
    if (chunks > 65535) return KB_ERR_UNSUPPORTED_SIZE;
    kb_launch(logprob_chunk_kernel, dim3(reports, chunks), dim3(REPORT_THREADS), 0, stream, logits, ld, V, rows, k, len, scratch);
    int rc = kb_launch_result();
    if (rc != 0) return rc;
    kb_launch(logprob_merge_kernel, dim3(reports), dim3(REPORT_THREADS), 0, stream, logits, ld, V, rows, tokens, tokens_by_row, k,
              chunks, (const float*)scratch, values, indices);
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

// The same noise in 32-bit arithmetic, within NOISE_SLACK of the 64-bit value over the whole range of u:
// below one half, log1pf keeps the relative precision of a small u; above, 1 - u is taken from the integer.
// It only decides which entries the 64-bit noise is computed for.
#define NOISE_SLACK 1e-3f
__device__ __forceinline__ float gumbel_noise_estimate(int i, unsigned long long seed) {
    const unsigned long long counter = ((unsigned long long)i + 1ull) * 0x9E3779B97F4A7C15ull;
    const unsigned long long word = splitmix_finalize(counter ^ seed);
    // u = (k + 0.5) / 2^52 and 1 - u = ((2^52 - 1 - k) + 0.5) / 2^52: whichever is at most one half, from the
    // integer, so that no 64-bit arithmetic is left in the estimate
    const unsigned long long k = word & ((1ull << 52) - 1ull);
    const bool low = k < (1ull << 51);
    const float t = ((float)(low ? k : (1ull << 52) - 1ull - k) + 0.5f) * 2.220446049250313e-16f;
    // -log(1 - t) for t in (0, 1/2]: the series where 1 - t would round the small t away (its next term is
    // below t^3 / 4 of the sum), the fast logarithm elsewhere (absolute error 2^-21 on a value of at least
    // 1 / 256); then the fast logarithm of that level: together some 1e-4, a tenth of NOISE_SLACK
    float level;
    if (low) level = t < 0.00390625f ? t * (1.0f + t * (0.5f + t * 0.33333334f)) : -__logf(1.0f - t);
    else level = -__logf(t);
    return -__logf(level);
}

// ---- stage 1 runs as a thread-block cluster per row: SAMPLE_CLUSTER blocks share the row's passes
// (each block owns a slice of the vocabulary) and combine their partial results through
// distributed shared memory, in rank order, so every block holds the same totals.
#define SAMPLE_CLUSTER 8
#define STAGE1_THREADS 512
#define STAGE1_WARPS (STAGE1_THREADS / 32)

// Two slots, used in turn: a reduction writes one slot, meets the others at one cluster barrier and
// reads theirs; the next reduction writes the other slot, so nobody overwrites what a slower block
// is still reading (it cannot be more than one reduction behind: the barrier in between).
struct ClusterScratch {
    float vals[2][16];  // this block's partial result of the reduction in progress
    int index[2];       // (argmax) the index that goes with vals[.][0]
    int turn;           // which slot the next reduction uses (the same in every block)
    float combined[16]; // the reduction's result, read from the other blocks by a few threads for all of this block's
    unsigned long long hist[2][256];  // (threshold search) this block's histogram of the round in progress, two slots as vals
    unsigned long long total[256];    // the cluster's histogram of the round
    unsigned long long above;         // the search's running weight above the prefix
    int digit;                        // the digit the round chose
    int reached;                      // whether the entries the search looked at weigh as much as the target
};

// Every block calls this with its partial results in mine->vals[0..count); on return all[k] holds
// op over the ranks, in rank order, the same in every block.  One cluster barrier and one of the block
// (the result's buffer is free again by then: the next reduction writes it behind its own cluster barrier).
template <int COUNT, typename Op>
__device__ __forceinline__ void cluster_combine(cg::cluster_group& cluster, ClusterScratch* mine, int slot, float (&all)[COUNT], Op op) {
    cluster.sync();  // every block's partials are in its shared memory
    // Thread k fetches value k of every rank (in rank order) and leaves the result in this block's own
    // shared memory; with every thread fetching every value, a block made 57,000 remote loads a round.
    if (threadIdx.x < COUNT) {
        float theirs[SAMPLE_CLUSTER];  // the loads go out together; the values are combined in rank order after
#pragma unroll
        for (unsigned rank = 0; rank < SAMPLE_CLUSTER; ++rank)
            theirs[rank] = rank < cluster.num_blocks() ? cluster.map_shared_rank(mine, rank)->vals[slot][threadIdx.x] : 0.0f;
        float acc = theirs[0];
#pragma unroll
        for (unsigned rank = 1; rank < SAMPLE_CLUSTER; ++rank)
            if (rank < cluster.num_blocks()) acc = op(acc, theirs[rank]);
        mine->combined[threadIdx.x] = acc;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < COUNT; ++k) all[k] = mine->combined[k];
}
// The slot this reduction uses; every thread of every block sees the same sequence of slots.
__device__ __forceinline__ int next_slot(int& turn) {
    const int slot = turn;
    turn ^= 1;
    return slot;
}

__device__ __forceinline__ float cluster_sum(cg::cluster_group& cluster, ClusterScratch* mine, int& turn, float v, float* scratch) {
    const int slot = next_slot(turn);
    v = block_sum(v, scratch);
    if (threadIdx.x == 0) mine->vals[slot][0] = v;
    float all[1];
    cluster_combine(cluster, mine, slot, all, [](float a, float b) { return a + b; });
    return all[0];
}
__device__ __forceinline__ float cluster_max(cg::cluster_group& cluster, ClusterScratch* mine, int& turn, float v, float* scratch) {
    const int slot = next_slot(turn);
    v = block_max(v, scratch);
    if (threadIdx.x == 0) mine->vals[slot][0] = v;
    float all[1];
    cluster_combine(cluster, mine, slot, all, [](float a, float b) { return fmaxf(a, b); });
    return all[0];
}
// First index of the maximum over the cluster's slices.
__device__ __forceinline__ int cluster_argmax(cg::cluster_group& cluster, ClusterScratch* mine, int& turn, BestF b, float* sv, int* si) {
    const int slot = next_slot(turn);
    b = block_argmax(b, sv, si);
    if (threadIdx.x == 0) { mine->vals[slot][0] = b.v; mine->index[slot] = b.i; }
    cluster.sync();
    BestF best{-INFINITY, 0x7fffffff};
    for (unsigned rank = 0; rank < cluster.num_blocks(); ++rank) {
        const ClusterScratch* theirs = cluster.map_shared_rank(mine, rank);
        if (better(theirs->vals[slot][0], theirs->index[slot], best.v, best.i)) { best.v = theirs->vals[slot][0]; best.i = theirs->index[slot]; }
    }
    cluster.sync();  // the last reduction of a row: nobody leaves while its shared memory is being read
    return best.i;
}

// Exact sum of one 64-bit integer per thread over the block and the cluster (through the histogram's bins 0..warps).
__device__ __forceinline__ unsigned long long cluster_sum_units(cg::cluster_group& cluster, ClusterScratch* mine, int& turn, unsigned long long v) {
    const int slot = next_slot(turn);
    unsigned long long* bins = mine->hist[slot];
    if (threadIdx.x == 0) bins[0] = 0;
    __syncthreads();
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    if ((threadIdx.x & 31) == 0) atomicAdd(&bins[0], v);
    cluster.sync();
    unsigned long long sum = 0;
    for (unsigned rank = 0; rank < cluster.num_blocks(); ++rank) sum += cluster.map_shared_rank(mine, rank)->hist[slot][0];
    return sum;
}

// Weights of the threshold search are integers, so that no order of addition matters: a count is 1, a
// probability is its value in units of 2^-40 (a row's sum stays far below 2^64).
__device__ __forceinline__ unsigned long long mass_units(float pv) { return (unsigned long long)(pv * 1099511627776.0f); }  // a power of two: exact

// Smallest 32-bit key u such that weight{ key_i > u, key_i >= lo_key } < target,
// where key_i are the bits of the non-negative floats p_i and weight is a count
// (use_sum = 0) or the sum of p_i in units of 2^-40 (use_sum = 1).  Radix descent, 8 bits a round (four
// rounds): every block builds the histogram of its slice [begin, end) in shared memory (one histogram a
// warp; lanes with the same digit add up among themselves first: most of a row shares a few exponents),
// thread t adds up bin t of all the cluster's blocks, a warp walks the 256 bins from the top, and all
// blocks return the same u.  Requires target > 0 and a block of at least 256 threads.
__device__ unsigned int select_key(cg::cluster_group& cluster, ClusterScratch* mine, int& turn, const float* __restrict__ p, int begin,
                                   int end, unsigned int lo_key, unsigned long long target, int use_sum,
                                   unsigned long long (*warp_hist)[256], bool* reached = nullptr) {
    // `reached` (an attempt over the entries from lo_key up only, which the caller chose above its real
    // floor): after the first round, which has weighed all of them, the search gives up if they do not
    // reach the target, and says so; every block of the cluster sees the same totals and decides alike.
    unsigned int prefix = 0;
    if (threadIdx.x == 0) mine->above = 0;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    for (int shift = 24; shift >= 0; shift -= 8) {
        const int slot = next_slot(turn);
        // a histogram a warp: its lanes with the same digit add up among themselves and one of them adds the
        // sum to the warp's bin, so no two threads ever meet at a bin (most of a row shares a few exponents,
        // and atomics on those few bins took most of a round)
        unsigned long long* hist = warp_hist[warp];
        for (int d = lane; d < 256; d += 32) hist[d] = 0;
        __syncwarp();
        const unsigned int high_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        // eight of a thread's values are loaded together and then taken in turn: a load between the turns
        // would wait behind the warp's meeting points, one memory round trip a value
        constexpr int BATCH = 8;
        for (int base = begin + (int)threadIdx.x; base - (int)threadIdx.x < end; base += BATCH * (int)blockDim.x) {  // every lane of a warp makes the same turns
            float batch[BATCH];
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int i = base + u * (int)blockDim.x;
                batch[u] = i < end ? p[i] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int i = base + u * (int)blockDim.x;
                const float pv = batch[u];
                const unsigned int key = __float_as_uint(pv);
                const bool in = i < end && key >= lo_key && (key & high_mask) == (prefix & high_mask);
                const unsigned int taking = __ballot_sync(0xffffffffu, in);
                if (taking == 0) continue;
                if (in) {
                    const unsigned int digit = (key >> shift) & 255u;
                    const unsigned int same = __match_any_sync(taking, digit);
                    unsigned long long weight;
                    if (use_sum) {
                        const unsigned long long units = mass_units(pv);
                        const unsigned int low = __reduce_add_sync(same, (unsigned int)(units & 0xFFFFFu));
                        const unsigned int high = __reduce_add_sync(same, (unsigned int)(units >> 20));
                        weight = ((unsigned long long)high << 20) + low;
                    } else {
                        weight = (unsigned long long)__popc(same);
                    }
                    if (lane == __ffs(same) - 1) hist[digit] += weight;
                }
                __syncwarp();  // the next turn's leaders may be other lanes
            }
        }
        __syncthreads();
        for (int d = threadIdx.x; d < 256; d += blockDim.x) {
            unsigned long long sum = 0;
#pragma unroll
            for (int w = 0; w < STAGE1_WARPS; ++w) sum += warp_hist[w][d];
            mine->hist[slot][d] = sum;
        }
        cluster.sync();  // every block's histogram is complete (and the block's own threads have met)
        for (int d = threadIdx.x; d < 256; d += blockDim.x) {
            unsigned long long theirs[SAMPLE_CLUSTER];  // the remote loads go out together
#pragma unroll
            for (unsigned rank = 0; rank < SAMPLE_CLUSTER; ++rank)
                theirs[rank] = rank < cluster.num_blocks() ? cluster.map_shared_rank(mine, rank)->hist[slot][d] : 0ull;
            unsigned long long sum = 0;
#pragma unroll
            for (unsigned rank = 0; rank < SAMPLE_CLUSTER; ++rank) sum += theirs[rank];
            mine->total[d] = sum;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // G(d) = above + sum_{e>d} total[e]; the smallest d with G(d) < target.  Lane l owns bins 8l..8l+7:
            // the weight above a lane's bins comes from a scan over the lanes, then the lane in whose bins
            // G falls below the target for the last time (going down) walks its eight bins.
            unsigned long long own = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) own += mine->total[8 * lane + e];
            unsigned long long higher = own;  // inclusive sum over lanes >= this one
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const unsigned long long other = __shfl_down_sync(0xffffffffu, higher, offset);
                if (lane + offset < 32) higher += other;
            }
            const unsigned long long above_lane = mine->above + higher - own;  // G(8l + 7): the weight above this lane's top bin
            if (lane == 0) mine->reached = mine->above + higher >= target;  // lane 0's sum runs over every bin
            // going down from bin 255, G grows; the walk stops at the first bin d where G(d - 1) >= target
            const bool stops_here = !(above_lane + own < target);  // G(8l - 1) >= target: the stop lies in this lane's bins or above
            const unsigned int stopping = __ballot_sync(0xffffffffu, stops_here);
            const int owner = stopping ? 31 - __clz(stopping) : 0;  // the highest such lane; none: the walk reaches bin 0
            if (lane == owner) {
                int d = 8 * lane + 7;
                unsigned long long g = above_lane;
                while (d > 0) {
                    const unsigned long long g_next = g + mine->total[d];  // G(d-1)
                    if (!(g_next < target)) break;
                    g = g_next;
                    --d;
                    if (d < 8 * lane && stopping) break;  // not reached: the stop lies within the lane's bins
                }
                mine->above = g;
                mine->digit = d;
            }
        }
        __syncthreads();
        if (reached != nullptr && shift == 24) {
            *reached = mine->reached != 0;
            if (!*reached) return 0;
        }
        prefix |= (unsigned int)mine->digit << shift;
    }
    return prefix;
}

// Sampling runs as three launches.  Stage 1 (a cluster of SAMPLE_CLUSTER blocks per row, several
// passes over the row): probabilities and the filters' threshold.  Stage 2 (SAMPLE_CHUNKS blocks
// per row): the noisy argmax, whose 64-bit logarithms are the expensive part, over a chunk of the
// vocabulary each.  Stage 3 (one warp per row): the best of the chunks, in chunk order.
#define SAMPLE_CHUNKS 32
#define SAMPLE_NOISE_THREADS 256
struct SampleRowState {
    unsigned int lo_key;  // keep p with bits >= lo_key (and p > 0)
    float kept;           // their sum
    int decided;          // 1: out[r] is final already (temperature 0, or everything filtered)
    int pad;
};

// logits: [n, V] fp32 (read only); work: [n, V] fp32 scratch (probabilities).
// Per row: temperature (0 = argmax), top_k (<=0 or >=V: off), top_p (>=1: off),
// min_p (<=0: off).  One cluster (of up to SAMPLE_CLUSTER blocks) per row.
__global__ void __launch_bounds__(STAGE1_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, float* __restrict__ work, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              SampleRowState* __restrict__ state, int* __restrict__ out) {
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float scratch[32];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ ClusterScratch mine;
    __shared__ unsigned long long warp_hist[STAGE1_WARPS][256];
    int turn = 0;

    const int blocks_per_row = (int)cluster.num_blocks();
    const int r = blockIdx.x / blocks_per_row;
    const int rank = (int)cluster.block_rank();
    const int per = (V + blocks_per_row - 1) / blocks_per_row;
    const int begin = rank * per;
    const int end = min(begin + per, V);
    const float* row = logits + (size_t)r * ld;
    const float T = temperature[r];

    auto plain_argmax = [&]() {
        BestF b{-INFINITY, 0x7fffffff};
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float v = row[i];
            if (better(v, i, b.v, b.i)) { b.v = v; b.i = i; }
        }
        const int index = cluster_argmax(cluster, &mine, turn, b, sv, si);
        if (rank == 0 && threadIdx.x == 0) {
            out[r] = index == 0x7fffffff ? 0 : index;
            state[r].decided = 1;
        }
    };
    if (T == 0.0f) {
        plain_argmax();
        return;
    }

    float* p = work + (size_t)r * V;
    // softmax(logits / T)
    float mx = -INFINITY;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) mx = fmaxf(mx, row[i] / T);
    mx = cluster_max(cluster, &mine, turn, mx, scratch);
    float sum = 0.0f;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) sum += expf(row[i] / T - mx);
    sum = cluster_sum(cluster, &mine, turn, sum, scratch);
    // min-p: keep p >= min_p * max p (sampler.py:1244-1249)
    const float mp = min_p[r];
    const float p_max = 1.0f / sum;  // exp(0) / sum
    const float floor_p = mp > 0.0f ? mp * p_max : 0.0f;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        float pv = expf(row[i] / T - mx) / sum;
        if (pv < floor_p) pv = 0.0f;
        p[i] = pv;
    }
    __syncthreads();

    unsigned int lo_key = 0;
    // top-k: keep p >= k-th largest (ties kept) (sampler.py:1259-1291)
    const int k = top_k[r];
    if (k > 0 && k < V) lo_key = select_key(cluster, &mine, turn, p, begin, end, lo_key, (unsigned long long)k, 0, warp_hist);
    // top-p: in descending order drop a token once the mass before it reaches
    // top_p * total (sampler.py:1349-1361); tokens tied with the last kept one stay.
    const float tp = top_p[r];
    if (tp < 1.0f) {
        // the mass that top-k left, in the search's own units
        unsigned long long units = 0;
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float pv = p[i];
            if (__float_as_uint(pv) >= lo_key) units += mass_units(pv);
        }
        const unsigned long long total = cluster_sum_units(cluster, &mine, turn, units);
        unsigned long long target = (unsigned long long)((double)tp * (double)total);
        if (target < 1) target = 1;
        // First among the entries of at least 1/65536 of the mass only (a few thousand of a language
        // model's row, so the rounds' passes over the row find few to weigh): where these reach the
        // target, the entries below them cannot move the threshold.  A distribution so flat that they do
        // not is searched again over everything.
        const unsigned int floor_key = __float_as_uint((float)((double)total * (1.0 / 65536.0) * (1.0 / 1099511627776.0)));
        bool reached = false;
        unsigned int u = 0;
        if (floor_key > lo_key) u = select_key(cluster, &mine, turn, p, begin, end, floor_key, target, 1, warp_hist, &reached);
        if (!reached) u = select_key(cluster, &mine, turn, p, begin, end, lo_key, target, 1, warp_hist);
        lo_key = u > lo_key ? u : lo_key;
    }
    // what is left; its sum renormalises the draw
    float kept = 0.0f;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float pv = p[i];
        if (pv > 0.0f && __float_as_uint(pv) >= lo_key) kept += pv;
    }
    kept = cluster_sum(cluster, &mine, turn, kept, scratch);
    if (!(kept > 0.0f)) {  // everything filtered: fall back to the argmax (sampler.py:1363-1378)
        plain_argmax();
        return;
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
    if (rank == 0 && threadIdx.x == 0) {
        state[r].lo_key = lo_key;
        state[r].kept = kept;
        state[r].decided = 0;
    }
}

// grid (rows, SAMPLE_CHUNKS): the best of log(p / kept) + noise over this block's chunk of the row
// (ties: the lower index), written to best_v / best_i [rows, SAMPLE_CHUNKS].
__global__ void __launch_bounds__(SAMPLE_NOISE_THREADS)
sample_noise_kernel(const float* __restrict__ work, int V, const SampleRowState* __restrict__ state,
                    const unsigned long long* __restrict__ seeds, double* __restrict__ best_v, int* __restrict__ best_i) {
    pdl_wait();
    __shared__ double dv[SAMPLE_NOISE_THREADS / 32];
    __shared__ int di[SAMPLE_NOISE_THREADS / 32];
    const int r = blockIdx.x;
    const SampleRowState st = state[r];
    if (st.decided) return;
    const float* p = work + (size_t)r * V;
    const int per = (V + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
    const int begin = blockIdx.y * per;
    const int end = min(begin + per, V);
    const unsigned long long seed = seeds[r];
    // The 64-bit logarithms are what this kernel's time goes to, and all but the chunk's few best entries
    // lose by far.  A first pass takes the chunk's largest value in 32-bit arithmetic, which is within
    // NOISE_SLACK of the 64-bit one for every entry; the second computes the 64-bit value only where the
    // 32-bit one comes within twice that of the largest, which the winner in 64-bit does by construction.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float fv[SAMPLE_NOISE_THREADS / 32];
    float near_best = -INFINITY;
    for (int i = begin + threadIdx.x; i < end; i += SAMPLE_NOISE_THREADS) {
        const float pv = p[i];
        if (pv > 0.0f && __float_as_uint(pv) >= st.lo_key) near_best = fmaxf(near_best, __logf(pv) + gumbel_noise_estimate(i, seed));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) near_best = fmaxf(near_best, __shfl_xor_sync(0xffffffffu, near_best, o));
    if (lane == 0) fv[warp] = near_best;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < SAMPLE_NOISE_THREADS / 32; ++w) near_best = fmaxf(near_best, fv[w]);
    const float bar = near_best - 2.0f * NOISE_SLACK - 1e-6f * fabsf(near_best);  // and the rounding of the 32-bit sum itself
    double best = -INFINITY;
    int best_index = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += SAMPLE_NOISE_THREADS) {
        const float pv = p[i];
        if (pv > 0.0f && __float_as_uint(pv) >= st.lo_key) {
            // (the row's log kept is the same for all: left out of the 32-bit values; keeping the first pass's
            // values in shared memory instead of computing them again gained 13 us at 64 unfiltered rows and
            // lost 10 at 64 filtered ones, whose blocks then share an SM with fewer others)
            if (__logf(pv) + gumbel_noise_estimate(i, seed) < bar) continue;
            const double v = (double)logf(pv / st.kept) + gumbel_noise(i, seed);
            if (v > best || (v == best && i < best_index)) { best = v; best_index = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_index, o);
        if (ov > best || (ov == best && oi < best_index)) { best = ov; best_index = oi; }
    }
    if (lane == 0) { dv[warp] = best; di[warp] = best_index; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SAMPLE_NOISE_THREADS / 32; ++w)
            if (dv[w] > best || (dv[w] == best && di[w] < best_index)) { best = dv[w]; best_index = di[w]; }
        best_v[(size_t)r * SAMPLE_CHUNKS + blockIdx.y] = best;
        best_i[(size_t)r * SAMPLE_CHUNKS + blockIdx.y] = best_index;
    }
}

// one warp per row: the best chunk (ties: the lower index)
__global__ void sample_pick_kernel(const SampleRowState* __restrict__ state, const double* __restrict__ best_v,
                                   const int* __restrict__ best_i, int* __restrict__ out) {
    pdl_wait();
    const int r = blockIdx.x;
    if (state[r].decided) return;
    const int lane = threadIdx.x;
    double best = lane < SAMPLE_CHUNKS ? best_v[(size_t)r * SAMPLE_CHUNKS + lane] : -INFINITY;
    int best_index = lane < SAMPLE_CHUNKS ? best_i[(size_t)r * SAMPLE_CHUNKS + lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_index, o);
        if (ov > best || (ov == best && oi < best_index)) { best = ov; best_index = oi; }
    }
    if (lane == 0) out[r] = best_index == 0x7fffffff ? 0 : best_index;
}

// Scratch floats kb_sample needs beyond the n * V probabilities.
KB_EXPORT int kb_sample_extra_floats(int n) { return n * (4 + 3 * SAMPLE_CHUNKS) + 8; }

// work: n * V + kb_sample_extra_floats(n) floats of scratch.
KB_EXPORT int kb_sample(const float* logits, int ld, float* work, int n, int V,
                        const float* temperature, const int* top_k, const float* top_p,
                        const float* min_p, const unsigned long long* seeds, int* out,
                        cudaStream_t stream) {
    if (n == 0) return 0;
    if (!logits || !work || !temperature || !top_k || !top_p || !min_p || !seeds || !out) return KB_ERR_NULL;
    if (V < 1 || V >= (1 << 24)) return KB_ERR_UNSUPPORTED_SIZE;  // counts are kept in fp32
    static_assert(SAMPLE_CHUNKS <= 32, "the last stage is one warp per row");
    // scratch after the probabilities, on 8-byte boundaries: per-row state, then the chunks' best values and indices
    size_t offset = ((size_t)n * V + 1) & ~(size_t)1;
    SampleRowState* state = reinterpret_cast<SampleRowState*>(work + offset);
    offset += (size_t)n * 4;
    double* best_v = reinterpret_cast<double*>(work + offset);
    offset += (size_t)n * SAMPLE_CHUNKS * 2;
    int* best_i = reinterpret_cast<int*>(work + offset);
    {
        cudaLaunchConfig_t config = {};
        // blocks per row: eight for up to 32 rows, fewer for more, so that the clusters fit the device at once
        const int per_row = n <= 32 ? SAMPLE_CLUSTER : (n <= 64 ? 4 : 2);
        config.gridDim = dim3(n * per_row);
        config.blockDim = dim3(STAGE1_THREADS);
        config.stream = stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = per_row;
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = 1;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attributes;
        config.numAttrs = 2;
        cudaLaunchKernelEx(&config, sample_kernel, logits, ld, work, V, temperature, top_k, top_p, min_p, state, out);
    }
    int rc = kb_launch_result();
    if (rc != 0) return rc;
    kb_launch(sample_noise_kernel, dim3(n, SAMPLE_CHUNKS), dim3(SAMPLE_NOISE_THREADS), 0, stream, (const float*)work, V,
              (const SampleRowState*)state, seeds, best_v, best_i);
    rc = kb_launch_result();
    if (rc != 0) return rc;
    kb_launch(sample_pick_kernel, dim3(n), dim3(32), 0, stream, (const SampleRowState*)state, (const double*)best_v, (const int*)best_i, out);
    return kb_launch_result();
}
