// Shared device helpers for the sm_100a kernels of this engine.
//
// Conventions
//  * Every entry point is extern "C", takes raw device pointers plus a stream, and
//    returns 0 or a cudaError_t / negative argument error.  The Python launcher checks
//    shapes before the call; kernels check indices that come from device data
//    (token ids, page numbers, state slots) and record the first bad one in a status
//    word instead of touching memory out of range.
//  * dtype codes: 0 = float32, 1 = bfloat16.
//  * Softmax, norms, rotation angles and the residual stream are 32-bit in both modes.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define IMPARO_DT_F32 0
#define IMPARO_DT_BF16 1

// status word layout: [0] = code (0 ok), [1] = which kernel, [2] = index, [3] = value
#define IMPARO_ST_TOKEN_RANGE 1
#define IMPARO_ST_PAGE_RANGE 2
#define IMPARO_ST_SLOT_RANGE 3
#define IMPARO_ST_WAIT_LIMIT 4

namespace imparo {

__device__ __forceinline__ void report(int* status, int code, int kernel, int index, int value) {
    if (status && atomicCAS(status, 0, code) == 0) {
        status[1] = kernel;
        status[2] = index;
        status[3] = value;
    }
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// additions depends only on blockDim, never on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        float t = lane < nw ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        float t = lane < nw ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// x / (1 + exp(-x))
__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

}  // namespace imparo

// ---- programmatic dependent launch ----------------------------------------------------
// Every kernel of this engine calls pdl_trigger() first and then pdl_wait(), before it reads
// or writes anything an earlier kernel may touch.  The trigger lets the next kernel's CTAs be
// scheduled as soon as this kernel's CTAs are all resident; the wait returns when the previous
// kernel has completed, and that kernel only completes after its own wait, so completion is
// ordered along the whole chain.  Several kernels of the chain are thus resident ahead of the
// running one, their launch latency and prologues hidden; the products use the time to request
// their weight tiles (which no kernel writes).  Without the launch attribute both are no-ops.
// Before its wait a kernel may read only what no kernel of the chain writes: weights, and the
// batch description of the step (positions, request of a token, portion starts, state slots,
// block tables), which the host copies to the device before the step's first kernel.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern "C" int imparo_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = imparo_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define IMPARO_CHECK_LAUNCH() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)
