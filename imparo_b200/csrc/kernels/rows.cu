// Row-wise kernels: embedding gather, RMS norm, SiLU-gate multiply, bias add.
//
// Formulas (zeraix/imparo): embedding rows unscaled (imparo-model/src/cpu_support.rs:327-342);
// RMS norm mean = sum(x^2)/width, scale = 1/sqrt(mean+eps), y = x*scale*w
// (imparo-cpu/src/ops.rs:6-22); silu(g)*u with SiLU on the gate (ops.rs:73-78,
// imparo-model/src/lfm2/workflow_cpu.rs:307-313).
#include "common.cuh"

namespace imparo {

// ---- embedding -----------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int width, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report(status, IMPARO_ST_TOKEN_RANGE, 1, t, id);
        id = 0;
    }
    const T* row = table + (size_t)id * width;
    float* o = out + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32(row[i]);
}

// ---- RMS norm ------------------------------------------------------------------------
// One block per output row.  rows == nullptr: output row r reads input row r; else input
// row rows[r].  The sum of squares is a fixed tree over blockDim threads, so a row's
// result never depends on which other rows are in the launch.
template <typename TOut>
__device__ __forceinline__ void store4(TOut* o, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* o, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* o, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <typename TOut>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const float* __restrict__ w, float eps, TOut* __restrict__ out,
                               int width) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
    TOut* o = out + (size_t)r * width;
    float ss = 0.f;
    if ((width & 3) == 0) {                       // 16-byte loads; the second pass re-reads from L1/L2
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)width + eps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            store4<TOut>(o + i, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TOut>(xr[i] * scale * w[i]);
}

// Many rows (a prompt portion) of a width that is a multiple of 128 up to 3,072 (the row must fit the registers): a warp per row, the row in
// registers (every load of the row in flight at once), sums by shuffles: one pass and no block-wide barrier.  The
// block-per-row kernel above spends its time in three barriers and a second pass over the row.
template <typename TOut, int NV>       // NV float4 per lane: width = 128 * NV
__global__ void __launch_bounds__(128)
rmsnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w, float eps,
                    TOut* __restrict__ out, int n_rows) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    constexpr int width = 128 * NV;
    float4 g[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) g[i] = __ldg(reinterpret_cast<const float4*>(w) + lane + 32 * i);
    pdl_wait();
    if (r >= n_rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * width);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = xr[lane + 32 * i];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TOut* o = out + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        store4<TOut>(o + 4 * (lane + 32 * i), v[i].x * scale * g[i].x, v[i].y * scale * g[i].y, v[i].z * scale * g[i].z,
                     v[i].w * scale * g[i].w);
}

// ---- stream += split partials, then RMS norm ----------------------------------------------
// A product that was cut along K leaves its partial results part[s][row][:] (s = 0..S-1) instead
// of adding them into the 32-bit stream itself.  This kernel adds them in split order (the same
// sum every time), writes the stream back, and — when out is given — norms the updated row in the
// same pass.  The reference fuses the same pair, residual add then norm
// (imparo-backend/src/lib.rs:2609-2623 add_rms_norm).
template <typename TOut>
__global__ void add_partials_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ part, int n_splits,
                                            size_t split_stride, const float* __restrict__ w, float eps,
                                            TOut* __restrict__ out, int width) {
    __shared__ float scratch[33];
    pdl_trigger();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * width;
    const float* pr = part + (size_t)r * width;
    float ss = 0.f;
    if ((width & 3) == 0 && (split_stride & 3) == 0 && width <= (int)blockDim.x * 4) {
        // A thread owns four columns and keeps them in registers.  The norm weight (written by no
        // kernel) is fetched before the wait; after it the row and all its partials are requested
        // at once, so the kernel costs one round trip to memory, a block sum and the stores.
        const int i = threadIdx.x * 4;
        const bool mine = i < width;
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mine && out) g = __ldg(reinterpret_cast<const float4*>(w + i));
        pdl_wait();
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mine) {
            v = *reinterpret_cast<const float4*>(xr + i);
            for (int s0 = 0; s0 < n_splits; s0 += 16) {
                float4 p[16];
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (s0 + u < n_splits) p[u] = __ldcg(reinterpret_cast<const float4*>(pr + (size_t)(s0 + u) * split_stride + i));
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (s0 + u < n_splits) { v.x += p[u].x; v.y += p[u].y; v.z += p[u].z; v.w += p[u].w; }
            }
            *reinterpret_cast<float4*>(xr + i) = v;
            ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        if (out == nullptr) return;
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)width + eps);
        if (mine) store4<TOut>(out + (size_t)r * width + i, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        return;
    }
    pdl_wait();
    if ((width & 3) == 0 && (split_stride & 3) == 0) {
        // 16-byte loads, and all of a chunk's split loads in flight before the (ordered) adds
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(xr + i);
            for (int s0 = 0; s0 < n_splits; s0 += 8) {
                float4 p[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (s0 + u < n_splits) p[u] = __ldcg(reinterpret_cast<const float4*>(pr + (size_t)(s0 + u) * split_stride + i));
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (s0 + u < n_splits) { v.x += p[u].x; v.y += p[u].y; v.z += p[u].z; v.w += p[u].w; }
            }
            *reinterpret_cast<float4*>(xr + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = xr[i];
            for (int s = 0; s < n_splits; ++s) v += pr[(size_t)s * split_stride + i];
            xr[i] = v;
            ss += v * v;
        }
    }
    if (out == nullptr) return;
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TOut* o = out + (size_t)r * width;
    __syncthreads();                                  // other threads' writes of this row (block scope)
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TOut>(xr[i] * scale * w[i]);
}

// ---- out[r, :] = x[rows[r], :] ---------------------------------------------------------------
// Rows of the 32-bit stream picked out (the last layer's feed-forward runs on the wanted rows only).
__global__ void gather_rows_f32_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                       float* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    const float* src = x + (size_t)rows[blockIdx.x] * width;
    float* dst = out + (size_t)blockIdx.x * width;
    if ((width & 3) == 0) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4)
            *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

// ---- out = sum of split partials ----------------------------------------------------------
// For a consumer that cannot read partials itself: out[i] = part[0][i] + part[1][i] + ... in order.
template <typename TOut>
__global__ void fold_partials_kernel(const float* __restrict__ part, int n_splits, size_t split_stride,
                                     TOut* __restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = s0 + u < n_splits ? __ldcg(part + (size_t)(s0 + u) * split_stride + i) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) if (s0 + u < n_splits) acc += v[u];
    }
    out[i] = from_f32<TOut>(acc);
}

// ---- silu(gate) * up ----------------------------------------------------------------
// gu: [T, 2F] rows = [gate | up]; out: [T, F]
template <typename T>
__global__ void swiglu_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int n_tok, int F) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_tok * F) return;
    const size_t t = i / F, f = i % F;
    const float g = to_f32(gu[t * 2 * F + f]);
    const float u = to_f32(gu[t * 2 * F + F + f]);
    out[i] = from_f32<T>(silu(g) * u);
}

// eight features per thread, 16-byte loads and stores (F a multiple of 8)
__global__ void swiglu_act_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int n_tok, int F) {
    pdl_trigger();
    pdl_wait();
    const int per_row = F >> 3;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_tok * per_row) return;
    const size_t t = i / per_row, f = (i % per_row) << 3;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * F + f);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + f);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 r;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 a = __bfloat1622float2(gp[k]), b = __bfloat1622float2(up[k]);
        rp[k] = __floats2bfloat162_rn(silu(a.x) * b.x, silu(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(out + t * F + f) = r;
}

// ---- out[t, :] += bias ----------------------------------------------------------------
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, int n_tok, int width) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_tok * width) return;
    out[i] = from_f32<T>(to_f32(out[i]) + bias[i % width]);
}

// ---- zero the state slots of requests that start in this step --------------------------------
// arena: every fixed-size state tensor of the model, [slots][floats per slot] each, one after the
// other; segments: per tensor (offset in the arena, floats per slot).  slots: the fresh slots of
// the step (a padded list: entries below 0 are skipped).  One block column per (tensor, slot).
__global__ void zero_state_slots_kernel(float* __restrict__ arena, const long long* __restrict__ segments,
                                        const int* __restrict__ slots, int n_slots_total, int* status) {
    pdl_trigger();
    const int seg = blockIdx.y, which = blockIdx.z;
    const int slot = slots[which];
    const long long off = segments[2 * seg], per = segments[2 * seg + 1];
    pdl_wait();
    if (slot < 0) return;
    if (slot >= n_slots_total) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && seg == 0) report(status, IMPARO_ST_SLOT_RANGE, 6, which, slot);
        return;
    }
    float* p = arena + off + (long long)slot * per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) p[i] = 0.f;
}

}  // namespace imparo

using namespace imparo;

extern "C" int imparo_zero_state_slots(float* arena, const long long* segments, int n_segments, long long max_per_slot,
                                       const int* slots, int n, int n_slots_total, int* status, cudaStream_t stream) {
    if (n <= 0 || n_segments <= 0) return 0;
    if (n > 65535 || n_segments > 65535) return -2;
    const int threads = 256;
    long long bx = (max_per_slot + threads * 4 - 1) / (threads * 4);
    if (bx < 1) bx = 1;
    if (bx > 64) bx = 64;
    launch(zero_state_slots_kernel, dim3((unsigned)bx, n_segments, n), dim3(threads), 0, stream, arena, segments, slots,
           n_slots_total, status);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// Programmatic dependent launch for every kernel of the engine: on by default.
static int g_pdl = 1;
extern "C" int imparo_pdl_enabled() { return g_pdl; }
extern "C" void imparo_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// ---- device timeline: host side (see common.cuh) -------------------------------------------
// buffer: device memory of (2 + 4 * capacity) 64-bit words.  Returns -1 when the library was
// built without IMPARO_TIMELINE.
extern "C" int imparo_timeline_start(unsigned long long* buffer, long long capacity) {
#ifdef IMPARO_TIMELINE
    if (buffer == nullptr || capacity <= 0) { g_timeline_host = nullptr; ++g_timeline_epoch; return 0; }
    const unsigned long long head[2] = {0ULL, (unsigned long long)capacity};
    cudaError_t e = cudaMemcpy(buffer, head, sizeof(head), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return (int)e;
    g_timeline_host = buffer;
    ++g_timeline_epoch;
    g_timeline_funcs.clear();
    return 0;
#else
    (void)buffer; (void)capacity;
    return -1;
#endif
}
// launches noted on the host since imparo_timeline_start (stream captures included), and the
// name of the i-th one
extern "C" long long imparo_timeline_launches() {
#ifdef IMPARO_TIMELINE
    return (long long)g_timeline_funcs.size();
#else
    return -1;
#endif
}
extern "C" int imparo_timeline_name(long long i, char* out, int n) {
#ifdef IMPARO_TIMELINE
    if (i < 0 || i >= (long long)g_timeline_funcs.size() || n <= 0) return -2;
    const char* name = nullptr;
    cudaError_t e = cudaFuncGetName(&name, g_timeline_funcs[(size_t)i]);
    if (e != cudaSuccess || name == nullptr) return (int)e;
    int k = 0;
    for (; k < n - 1 && name[k]; ++k) out[k] = name[k];
    out[k] = 0;
    return 0;
#else
    (void)i; (void)out; (void)n;
    return -1;
#endif
}

extern "C" int imparo_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                                   int n_tok, int width, int vocab, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == IMPARO_DT_F32)
        launch(embed_gather_kernel<float>, dim3(n_tok), dim3(threads), 0, stream, (const float*)table, ids, out, width, vocab, status);
    else if (table_dtype == IMPARO_DT_BF16)
        launch(embed_gather_kernel<__nv_bfloat16>, dim3(n_tok), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, out, width, vocab, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_rmsnorm(const float* x, const int* rows, const float* w, float eps, void* out,
                              int out_dtype, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (out_dtype != IMPARO_DT_F32 && out_dtype != IMPARO_DT_BF16) return -1;
    if (n_rows >= 256 && width % 128 == 0 && width <= 3072 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
        // a prompt portion: a warp per row
        const dim3 grid((n_rows + 3) / 4), block(128);
#define IMPARO_RN(T_, NV_) launch(rmsnorm_rows_kernel<T_, NV_>, grid, block, 0, stream, x, rows, w, eps, (T_*)out, n_rows)
#define IMPARO_RNV(T_) do { switch (width / 128) { \
            case 1: IMPARO_RN(T_, 1); break; case 2: IMPARO_RN(T_, 2); break; case 3: IMPARO_RN(T_, 3); break; case 4: IMPARO_RN(T_, 4); break; \
            case 5: IMPARO_RN(T_, 5); break; case 6: IMPARO_RN(T_, 6); break; case 7: IMPARO_RN(T_, 7); break; case 8: IMPARO_RN(T_, 8); break; \
            case 12: IMPARO_RN(T_, 12); break; case 16: IMPARO_RN(T_, 16); break; case 24: IMPARO_RN(T_, 24); break; \
            default: goto general; } } while (0)
        if (out_dtype == IMPARO_DT_F32) IMPARO_RNV(float); else IMPARO_RNV(__nv_bfloat16);
#undef IMPARO_RNV
#undef IMPARO_RN
        IMPARO_CHECK_LAUNCH();
        return 0;
    }
general:
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (out_dtype == IMPARO_DT_F32)
        launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, rows, w, eps, (float*)out, width);
    else if (out_dtype == IMPARO_DT_BF16)
        launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, rows, w, eps, (__nv_bfloat16*)out, width);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_swiglu_act(const void* gu, void* out, int dtype, int n_tok, int F, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    const size_t n = (size_t)n_tok * F;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == IMPARO_DT_F32)
        launch(swiglu_act_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, n_tok, F);
    else if (dtype == IMPARO_DT_BF16 && (F & 7) == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0)
        launch(swiglu_act_bf16x8_kernel, dim3((unsigned)((n / 8 + threads - 1) / threads)), dim3(threads), 0, stream,
               (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tok, F);
    else if (dtype == IMPARO_DT_BF16)
        launch(swiglu_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tok, F);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_add_bias(void* out, int dtype, const float* bias, int n_tok, int width, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    const size_t n = (size_t)n_tok * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == IMPARO_DT_F32)
        launch(add_bias_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)out, bias, n_tok, width);
    else if (dtype == IMPARO_DT_BF16)
        launch(add_bias_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, bias, n_tok, width);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// x[r, :] += sum over s of part[s][r][:] (in order), and out = rms_norm(x) when out is not null.
extern "C" int imparo_gather_rows_f32(const float* x, const int* rows, float* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    launch(gather_rows_f32_kernel, dim3(n_rows), dim3(width >= 1024 ? 256 : 128), 0, stream, x, rows, out, width);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_fold_partials(const float* part, int n_splits, long long split_stride, void* out, int out_dtype,
                                    long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n_splits < 1 || split_stride < n) return -2;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (out_dtype == IMPARO_DT_F32)
        launch(fold_partials_kernel<float>, dim3(blocks), dim3(threads), 0, stream, part, n_splits, (size_t)split_stride, (float*)out, (size_t)n);
    else if (out_dtype == IMPARO_DT_BF16)
        launch(fold_partials_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, part, n_splits, (size_t)split_stride,
               (__nv_bfloat16*)out, (size_t)n);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_add_partials_rmsnorm(float* x, const float* part, int n_splits, long long split_stride,
                                           const float* w, float eps, void* out, int out_dtype, int n_rows, int width,
                                           cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    // a thread per four columns where the row fits a block (the kernel's one-pass form): 1,536 columns take 384
    // threads, not 256 and a second trip
    int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if ((width & 3) == 0 && width > threads * 4 && width <= 4096) threads = (width / 4 + 31) / 32 * 32;
    if (out == nullptr || out_dtype == IMPARO_DT_F32)
        launch(add_partials_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, part, n_splits, (size_t)split_stride,
               w, eps, (float*)out, width);
    else if (out_dtype == IMPARO_DT_BF16)
        launch(add_partials_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, part, n_splits,
               (size_t)split_stride, w, eps, (__nv_bfloat16*)out, width);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}
