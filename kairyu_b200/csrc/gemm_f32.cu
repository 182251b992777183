// y[M,N] = x[M,K] . W[N,K]^T (+ bias[N]) in true fp32: plain FMA on CUDA cores,
// no tensor cores and no reduced-precision mode.  Each output element adds its terms
// in order of k, 256 at a time into one accumulator whose sums are then added in
// order into a second (a sum of 8,192 terms carries the rounding of 256 + 32
// additions, not of 8,192), so a row's result does not depend on M or on which tile
// it falls in: the 32-bit path is bit-stable however a prompt is cut into steps.
#include "common.cuh"

#define F32_BM 64
#define F32_BN 64
#define F32_BK 16
#define F32_SUM_BLOCK 256  // terms a first-level accumulator takes before it is added to the second

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, int ldw,
                const float* __restrict__ bias, float* __restrict__ y, int ldy, int M, int N, int K) {
    pdl_wait();
    __shared__ float As[F32_BK][F32_BM + 1];
    __shared__ float Bs[F32_BK][F32_BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15;
    const int ty = tid >> 4;
    const int m0 = blockIdx.y * F32_BM;
    const int n0 = blockIdx.x * F32_BN;

    float acc[4][4], total[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = total[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += F32_BK) {
        if (k0 > 0 && k0 % F32_SUM_BLOCK == 0) {  // a block of 256 terms is complete
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    total[i][j] += acc[i][j];
                    acc[i][j] = 0.0f;
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4;
            const int c = idx & 15;
            const int k = k0 + c;
            const int m = m0 + r;
            const int n = n0 + r;
            As[c][r] = (m < M && k < K) ? x[(size_t)m * ldx + k] : 0.0f;
            Bs[c][r] = (n < N && k < K) ? w[(size_t)n * ldw + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < F32_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = total[i][j] + acc[i][j];
            if (bias) v += bias[n];
            y[(size_t)m * ldy + n] = v;
        }
    }
}

KB_EXPORT int kb_gemm_f32(const float* x, int ldx, const float* w, int ldw, const float* bias,
                          float* y, int ldy, int M, int N, int K, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (!x || !w || !y) return KB_ERR_NULL;
    if (K < 1) return KB_ERR_BAD_ARG;
    dim3 grid((N + F32_BN - 1) / F32_BN, (M + F32_BM - 1) / F32_BM);
    if (grid.y > 65535) return KB_ERR_UNSUPPORTED_SIZE;
    kb_launch(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, x, ldx, w, ldw, bias, y, ldy, M, N, K);
    return kb_launch_result();
}
