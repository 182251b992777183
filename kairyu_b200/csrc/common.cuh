// Shared helpers of the sm_100a kernels: element conversion, reductions with a
// fixed order, the C export macro and launch checking.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KB_EXPORT extern "C" __attribute__((visibility("default")))

// Return codes of every exported entry point: 0 ok, >0 a cudaError_t from the
// launch, <0 an argument this kernel refuses (the Python side turns the code
// into a message).
#define KB_ERR_BAD_ARG (-1)
#define KB_ERR_UNSUPPORTED_SIZE (-2)
#define KB_ERR_NULL (-3)

static inline int kb_launch_result() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  Every kernel of this package is launched with the
// attribute below and calls pdl_wait() before it reads or writes anything that depends on
// the kernel before it (pdl_wait blocks until that kernel has finished and its writes are
// visible).  The attribute lets a kernel's blocks be scheduled while the previous kernel
// drains, so launch latency, set-up and, for the weight-streaming products, the first weight
// loads overlap its tail.
//
// pdl_trigger() (griddepcontrol.launch_dependents) lets the NEXT kernel's blocks be scheduled
// as soon as every block of this one has called it.  Only kernels that leave most of the SMs'
// resources free call it, and they call it first thing: the small-grid kernels (norm, position
// encoding, the merge of decode attention) and the register-only skinny product, whose followers then sit resident and have
// their first weights on the way.  Measured on the decode step (batch 8, 32 layers): -2.4 %.
// A trigger in the kernels that fill shared memory (the tcgen05 product, decode attention)
// made the step slower, wherever in the kernel it stood, so they have none.
// What a kernel reads of the step's description (positions, rows, lengths, block tables: written by
// the host's copy before the step's first kernel) and of the weights does not depend on the kernel
// before it, so those loads stand ahead of pdl_wait() where they start a chain of dependent loads.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline void kb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);  // the error, if any, is read by kb_launch_result()
}

// Bits of the device-side error word that indexing kernels set instead of
// touching memory outside their tensors.
#define KB_FLAG_BAD_PAGE 1
#define KB_FLAG_BAD_TOKEN 2
#define KB_FLAG_BAD_ROW 4
#define KB_FLAG_BAD_POS 8

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block in a fixed order (warp butterflies, then warp 0 over the
// per-warp partials): the result depends only on blockDim, never on the grid.
// `scratch` holds at least 32 floats.  Every thread gets the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? scratch[lane] : 0.0f;
    total = warp_sum(total);
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? scratch[lane] : -INFINITY;
    total = warp_max(total);
    return total;
}

// Waits on barriers are bounded by time, not by a number of polls: two seconds on the GPU's
// nanosecond timer, whatever the clocks are and however a profiler serialises the roles of a
// block (a poll count that is generous at full speed ran out under a profiler's replay).
#define KB_WAIT_LIMIT_NS 2000000000ull
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
