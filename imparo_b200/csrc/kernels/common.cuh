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
// The same for results that are rounded to bfloat16 at once: the exponential and the division by their
// approximate instructions (a few units in the last place of 32-bit, far below the rounding that follows).
__device__ __forceinline__ float silu_bf16(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

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
#ifndef IMPARO_TIMELINE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// A kernel that wants the SMs to itself for a while triggers late: timeline_begin() where it
// starts, pdl_trigger_late() where the dependents may come.
__device__ __forceinline__ void pdl_trigger_late() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Two kernels of the chain that touch different rows may run side by side (the prompt portions' attention and the decode
// rows' of one step).  The first then lets its dependents come only after its own wait (timeline_begin(), pdl_wait(),
// pdl_trigger_late()), so that the second, which starts with pdl_no_wait(), finds everything before the first complete;
// and the second ends with pdl_wait_at_end() in one thread of every CTA: it completes only after the first, and the
// chain behind it stays ordered.
__device__ __forceinline__ void pdl_no_wait() {}
__device__ __forceinline__ void pdl_wait_at_end() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void timeline_begin() {}
__device__ __forceinline__ void timeline_mark(int) {}
#else
// ---- device timeline (a build of its own, -DIMPARO_TIMELINE) ----------------------------
// Thread 0 of block (0,0,0) of every launch takes the next record of a device buffer and stamps
// the global nanosecond timer when the kernel's first block starts (at pdl_trigger), when its
// wait on the previous kernel returns (at pdl_wait) and at up to two marks of the kernel's own.
// buffer: [0] next record, [1] capacity, then records of four 64-bit words.  Records are taken in
// launch order: a kernel's dependents cannot start before its blocks have all passed pdl_trigger.
// Each translation unit holds its own copy of the buffer address (set at its first launch after
// imparo_timeline_start); the host list of launched functions is shared.
#include <vector>
static __device__ unsigned long long* g_timeline = nullptr;
inline unsigned long long* g_timeline_host = nullptr;
inline int g_timeline_epoch = 0;
inline std::vector<const void*> g_timeline_funcs;
static int g_timeline_bound = -1;

__device__ __forceinline__ unsigned long long timeline_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ int* timeline_slot() { __shared__ int slot; return &slot; }
__device__ __forceinline__ bool timeline_thread() {
    return g_timeline != nullptr && threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
}
__device__ __forceinline__ void timeline_stamp(int word) {
    const int slot = *timeline_slot();
    if (slot >= 0) g_timeline[2 + (size_t)slot * 4 + word] = timeline_ns();
}
__device__ __forceinline__ void timeline_begin() {
    if (timeline_thread()) {
        const unsigned long long slot = atomicAdd(g_timeline, 1ULL);
        *timeline_slot() = slot < g_timeline[1] ? (int)slot : -1;
        timeline_stamp(0);
    }
}
__device__ __forceinline__ void pdl_trigger() {
    timeline_begin();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_trigger_late() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (timeline_thread()) timeline_stamp(1);
}
__device__ __forceinline__ void pdl_no_wait() { if (timeline_thread()) timeline_stamp(1); }
__device__ __forceinline__ void pdl_wait_at_end() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// which = 0 or 1; call it from ONE thread of the launch's blocks; only block (0,0,0) records
__device__ __forceinline__ void timeline_mark(int which) {
    if (g_timeline != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) timeline_stamp(2 + which);
}
// host: remember the launched function and make sure this unit knows the buffer
static inline cudaError_t timeline_note(const void* kernel) {
    if (g_timeline_host == nullptr) return cudaSuccess;
    if (g_timeline_bound != g_timeline_epoch) {
        cudaError_t e = cudaMemcpyToSymbol(g_timeline, &g_timeline_host, sizeof(g_timeline_host));
        if (e != cudaSuccess) return e;
        g_timeline_bound = g_timeline_epoch;
    }
    g_timeline_funcs.push_back(kernel);
    return cudaSuccess;
}
#endif
#ifndef IMPARO_TIMELINE
static inline cudaError_t timeline_note(const void*) { return cudaSuccess; }
#endif

extern "C" int imparo_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    {
        cudaError_t e = timeline_note(reinterpret_cast<const void*>(kernel));
        if (e != cudaSuccess) return e;
    }
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
