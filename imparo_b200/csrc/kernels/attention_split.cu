// Split-key attention for single query tokens (decode rows): the keys of one request are
// cut into fixed chunks, one CTA per (chunk, kv head, query token) computes an unnormalised
// partial result for all query heads of the group at once (keys and values are read once
// per group, not once per head), and a second kernel combines the chunks in order.
//
// The reference decodes the same way over its quantised cache: key ranges -> partials ->
// a deterministic combine (imparo-cuda/native/sm80/attention_decode_vec_d64_q8.cuh:270,475).
// Scores, softmax and the combine are 32-bit; the split is a function of the chunk size
// alone, which the launcher derives from the table width, never from arrival order.
//
// Scratch: part_acc [tokens, heads, splits, head] and part_ml [tokens, heads, splits, 2]
// (float32), owned by the caller.
#include "common.cuh"

namespace imparo {

constexpr int SPLIT_WARPS = 4;
constexpr int SPLIT_MAX_HEAD = 256;

template <typename T> struct KVec;
template <> struct KVec<float> { using type = float4; static constexpr int N = 4; };
template <> struct KVec<__nv_bfloat16> { using type = uint4; static constexpr int N = 8; };

template <int G>
__device__ __forceinline__ void dot_group(const float4& k, const float* q, int hd, int off, float (&s)[G]) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float4 qv = *reinterpret_cast<const float4*>(q + g * hd + off);
        s[g] += k.x * qv.x + k.y * qv.y + k.z * qv.z + k.w * qv.w;
    }
}
template <int G>
__device__ __forceinline__ void dot_group(const uint4& k, const float* q, int hd, int off, float (&s)[G]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&k);
    const float2 k0 = __bfloat1622float2(p[0]), k1 = __bfloat1622float2(p[1]);
    const float2 k2 = __bfloat1622float2(p[2]), k3 = __bfloat1622float2(p[3]);
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float4 qa = *reinterpret_cast<const float4*>(q + g * hd + off);
        const float4 qb = *reinterpret_cast<const float4*>(q + g * hd + off + 4);
        s[g] += k0.x * qa.x + k0.y * qa.y + k1.x * qa.z + k1.y * qa.w + k2.x * qb.x + k2.y * qb.y + k3.x * qb.z + k3.y * qb.w;
    }
}

__device__ __forceinline__ void unpack(const float4& v, float* o) { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
__device__ __forceinline__ void unpack(const uint4& v, float* o) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(p[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}

// dynamic shared memory layout (floats):
//   qs   [G][hd]                 the group's queries
//   ps   [WARPS][G][32]          a warp's probabilities for its 32 keys
//   rows [WARPS][32] (int)       their cache rows
//   wm, wl [WARPS][G]            per-warp running max / sum
//   wacc [WARPS][KPI][G][hd]     per-warp, per-lane-group accumulators (KPI = keys per load instruction)
// The arithmetic reads global memory in batches of independent loads.  (Staging the loads
// through shared memory with cp.async was tried and changed nothing: this kernel is bound by
// instruction issue; its tensor-core version is attn_decode_mma_kernel in attention_prefill.cu.)
template <typename T, int G>
__global__ void __launch_bounds__(SPLIT_WARPS * 32)
attn_split_partial_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                          const int* __restrict__ positions, const int* __restrict__ item_of_token,
                          const int* __restrict__ table, int max_blocks, int page_size, int n_pages, int window,
                          float scale, float* __restrict__ part_acc, float* __restrict__ part_ml,
                          int nh, int nkv, int hd, int chunk, int n_splits, int* status) {
    extern __shared__ __align__(16) float smem[];
    pdl_trigger();
    pdl_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* qs = smem;
    float* ps = qs + G * hd;
    int* rows = reinterpret_cast<int*>(ps + SPLIT_WARPS * G * 32);
    float* wm = reinterpret_cast<float*>(rows + SPLIT_WARPS * 32);
    float* wl = wm + SPLIT_WARPS * G;
    float* wacc = wl + SPLIT_WARPS * G;

    const int pos = positions[t];
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int begin = max(lo, split * chunk), end = min(pos + 1, (split + 1) * chunk);
    const int h0 = kvh * G;
    const size_t part_base = ((size_t)t * nh + h0) * n_splits + split;     // + g * n_splits
    if (begin >= end) {
        if (threadIdx.x < G) {
            part_ml[(part_base + (size_t)threadIdx.x * n_splits) * 2] = -INFINITY;
            part_ml[(part_base + (size_t)threadIdx.x * n_splits) * 2 + 1] = 0.f;
        }
        return;
    }
    for (int i = threadIdx.x; i < G * hd; i += blockDim.x) qs[i] = to_f32(q[((size_t)t * nh + h0) * hd + i]);
    __syncthreads();

    const int* tab = table + (size_t)item_of_token[t] * max_blocks;
    const size_t kvw = (size_t)nkv * hd;
    using V = typename KVec<T>::type;
    constexpr int VN = KVec<T>::N;
    // Values: a row of hd elements is read by LPR lanes with one vector each (VPL vectors when
    // the row has more than 32 vectors), so one load instruction of the warp covers KPI keys.
    const int vecs = hd / VN;
    const int LPR = vecs < 32 ? vecs : 32;            // lanes per row
    const int VPL = (vecs + LPR - 1) / LPR;           // vectors per lane: 1, or 2 for float32 heads above 128 (the
                                                      // second exists for lanes with lig + LPR < vecs only)
    const int KPI = 32 / LPR;                         // keys per instruction
    const int grp = lane / LPR, lig = lane % LPR;     // lane group = which key, lane in group = which vector
    const bool pv_lane = grp < KPI;
    constexpr int ACC = 8;                            // VN * VPL <= 8
    float acc[G][ACC];
    float m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[g][i] = 0.f;
    }
    float* my_ps = ps + warp * G * 32;
    int* my_rows = rows + warp * 32;

    auto lookup = [&](int j) -> int {
        if (j >= end) return -1;
        const int blk = j / page_size;
        const int page = blk < max_blocks ? tab[blk] : -1;
        if (page < 0 || page >= n_pages) { report(status, IMPARO_ST_PAGE_RANGE, 5, t, page); return -1; }
        return page * page_size + (j % page_size);
    };

    for (int base = begin + warp * 32; base < end; base += SPLIT_WARPS * 32) {
        const int j = base + lane;
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
        const int rowi = lookup(j);
        {
            if (rowi >= 0) {
                const V* kp = reinterpret_cast<const V*>(k_cache + (size_t)rowi * kvw + (size_t)kvh * hd);
                // eight independent 16-byte loads in flight before any arithmetic
                for (int c0 = 0; c0 < vecs; c0 += 8) {
                    V kv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (c0 + u < vecs) kv[u] = kp[c0 + u];
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (c0 + u < vecs) dot_group<G>(kv[u], qs, hd, (c0 + u) * VN, s);
                }
            }
        }
        my_rows[lane] = rowi;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float sg = rowi >= 0 ? s[g] * scale : -INFINITY;
            const float m_new = fmaxf(m[g], warp_max(sg));
            float p = 0.f, corr = 1.f;
            if (m_new != -INFINITY) {
                p = rowi >= 0 ? expf(sg - m_new) : 0.f;
                corr = m[g] == -INFINITY ? 0.f : expf(m[g] - m_new);
            }
            l[g] = l[g] * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < ACC; ++i) acc[g][i] *= corr;
            m[g] = m_new;
            my_ps[g * 32 + lane] = p;
        }
        __syncwarp();
        const int cnt = min(32, end - base);
        // all loads of a round are independent of the arithmetic: the compiler keeps several
        // rounds in flight
        // four rounds of value loads in flight at a time; a dead lane reads row 0 (always
        // mapped memory) and contributes with probability 0
        for (int r0 = 0; r0 * KPI < cnt; r0 += 4) {
            V vv[4][2];
            int rjs[4], jjs[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int jj = (r0 + u) * KPI + grp;
                const bool live = pv_lane && jj < cnt;
                const int rj = live ? my_rows[jj] : -1;
                rjs[u] = rj;
                jjs[u] = jj & 31;
                const V* vp = reinterpret_cast<const V*>(v_cache + (size_t)(rj < 0 ? 0 : rj) * kvw + (size_t)kvh * hd);
                vv[u][0] = vp[lig];
                if (VPL > 1 && lig + LPR < vecs) vv[u][1] = vp[lig + LPR];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float v[ACC];
                unpack(vv[u][0], v);
                if (VPL > 1 && lig + LPR < vecs) unpack(vv[u][1], v + VN); else { for (int i = VN; i < ACC; ++i) v[i] = 0.f; }
                if (rjs[u] < 0) {             // whatever row 0 holds must not reach the sum (0 * inf)
#pragma unroll
                    for (int i = 0; i < ACC; ++i) v[i] = 0.f;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pj = rjs[u] < 0 ? 0.f : my_ps[g * 32 + jjs[u]];
#pragma unroll
                    for (int i = 0; i < ACC; ++i) acc[g][i] += pj * v[i];
                }
            }
        }
        __syncwarp();
    }
    // fold the lane groups and the warps, in that order
    float* my_acc = wacc + (size_t)(warp * KPI + (pv_lane ? grp : 0)) * G * hd;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { wm[warp * G + g] = m[g]; wl[warp * G + g] = l[g]; }
        if (pv_lane) {
            for (int u = 0; u < VPL; ++u)
#pragma unroll
                for (int i = 0; i < ACC; ++i)
                    if (i < VN && lig + u * LPR < vecs) my_acc[(size_t)g * hd + (lig + u * LPR) * VN + i] = acc[g][u * VN + i];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
        const int g = idx / hd, d = idx % hd;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < SPLIT_WARPS; ++w) M = fmaxf(M, wm[w * G + g]);
        float a = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < SPLIT_WARPS; ++w) {
                const float mw = wm[w * G + g];
                const float f = mw == -INFINITY ? 0.f : expf(mw - M);
                float aw = 0.f;
                for (int k = 0; k < KPI; ++k) aw += wacc[((size_t)(w * KPI + k) * G + g) * hd + d];
                a += aw * f;
                L += wl[w * G + g] * f;
            }
        }
        const size_t pb = part_base + (size_t)g * n_splits;
        part_acc[pb * hd + d] = a;
        if (d == 0) { part_ml[pb * 2] = M; part_ml[pb * 2 + 1] = L; }
    }
}

// One block per (token, head): fold the splits in order.  The splits' (max, sum) pairs go
// through shared memory and the first sixteen splits' accumulators are requested at the same
// time, so the usual launch costs one round trip to memory.
constexpr int COMBINE_MAX_SPLITS = 2048;
template <typename T>
__global__ void attn_split_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                          T* __restrict__ out, int hd, int n_splits) {
    __shared__ float f_s[COMBINE_MAX_SPLITS];             // exp(max_s - M), 0 for an empty split
    __shared__ float l_s[COMBINE_MAX_SPLITS];
    __shared__ float m_all;
    pdl_trigger();
    pdl_wait();
    const size_t th = blockIdx.x;                         // token * nh + head
    const float* ml = part_ml + th * n_splits * 2;
    const float* acc = part_acc + th * n_splits * hd;
    const int d0 = threadIdx.x;
    float pa[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) pa[u] = (u < n_splits && d0 < hd) ? __ldcg(acc + (size_t)u * hd + d0) : 0.f;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(ml) + s);
        f_s[s] = v.x;
        l_s[s] = v.y;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int s = threadIdx.x; s < n_splits; s += 32) if (l_s[s] > 0.f) M = fmaxf(M, f_s[s]);
        M = warp_max(M);
        if (threadIdx.x == 0) m_all = M;
    }
    __syncthreads();
    const float M = m_all;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) f_s[s] = l_s[s] > 0.f ? expf(f_s[s] - M) : 0.f;
    __syncthreads();
    for (int d = d0; d < hd; d += blockDim.x) {
        float a = 0.f, L = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 16) {
            if (s0 > 0 || d != d0) {
#pragma unroll
                for (int u = 0; u < 16; ++u) pa[u] = s0 + u < n_splits ? __ldcg(acc + (size_t)(s0 + u) * hd + d) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                if (s0 + u < n_splits && l_s[s0 + u] > 0.f) {
                    a += pa[u] * f_s[s0 + u];
                    L += l_s[s0 + u] * f_s[s0 + u];
                }
            }
        }
        out[th * hd + d] = from_f32<T>(L > 0.f ? a / L : 0.f);
    }
}

template <typename T, int G>
int launch_partial(const void* q, const void* k_cache, const void* v_cache, const int* positions, const int* item_of_token,
                   const int* table, int max_blocks, int page_size, int n_pages, int window, float scale,
                   float* part_acc, float* part_ml, int n_tok, int nh, int nkv, int hd, int chunk, int n_splits,
                   int* status, cudaStream_t stream) {
    const int vecs = hd / KVec<T>::N, lpr = vecs < 32 ? vecs : 32, kpi = 32 / lpr;
    const size_t smem = sizeof(float) * ((size_t)G * hd + SPLIT_WARPS * G * 32 + SPLIT_WARPS * 32 + 2 * SPLIT_WARPS * G +
                                         (size_t)SPLIT_WARPS * kpi * G * hd);
    auto kern = attn_split_partial_kernel<T, G>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_splits, nkv, n_tok);
    launch(kern, grid, dim3(SPLIT_WARPS * 32), smem, stream, (const T*)q, (const T*)k_cache, (const T*)v_cache, positions, item_of_token,
           table, max_blocks, page_size, n_pages, window, scale, part_acc, part_ml,
           nh, nkv, hd, chunk, n_splits, status);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

template <typename T>
int dispatch_group(int G, const void* q, const void* k_cache, const void* v_cache, const int* positions, const int* item_of_token,
                   const int* table, int max_blocks, int page_size, int n_pages, int window, float scale,
                   float* part_acc, float* part_ml, int n_tok, int nh, int nkv, int hd, int chunk, int n_splits,
                   int* status, cudaStream_t stream) {
#define IMPARO_G(g) case g: return launch_partial<T, g>(q, k_cache, v_cache, positions, item_of_token, table, max_blocks, page_size, \
        n_pages, window, scale, part_acc, part_ml, n_tok, nh, nkv, hd, chunk, n_splits, status, stream)
    switch (G) { IMPARO_G(1); IMPARO_G(2); IMPARO_G(3); IMPARO_G(4); IMPARO_G(5); IMPARO_G(6); IMPARO_G(7); IMPARO_G(8); }
#undef IMPARO_G
    return -8;
}

}  // namespace imparo

using namespace imparo;

// Returns -8 when the group size (heads / kv heads) is above 8: the caller then uses the
// general kernel.  n_tok must not exceed 65535 (grid z).
extern "C" int imparo_paged_attention_split(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                            const int* positions, const int* item_of_token,
                                            const int* table, int max_blocks, int page_size, int n_pages,
                                            int window, float scale, void* out, float* part_acc, float* part_ml,
                                            int n_tok, int nh, int nkv, int hd, int chunk, int n_splits,
                                            int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd < 16 || hd > SPLIT_MAX_HEAD || hd % 16 != 0) return -3;
    if (nkv <= 0 || nh % nkv != 0) return -5;
    if (n_tok > 65535 || nkv > 65535 || chunk < 32 || n_splits < 1 || n_splits > COMBINE_MAX_SPLITS) return -2;
    // the chunks must cover every position a table of this width can hold, or keys would be dropped silently
    if ((long long)chunk * n_splits < (long long)max_blocks * page_size) return -2;
    const int G = nh / nkv;
    int rc;
    if (dtype == IMPARO_DT_F32)
        rc = dispatch_group<float>(G, q, k_cache, v_cache, positions, item_of_token, table, max_blocks, page_size, n_pages,
                                   window, scale, part_acc, part_ml, n_tok, nh, nkv, hd, chunk, n_splits, status, stream);
    else if (dtype == IMPARO_DT_BF16)
        rc = dispatch_group<__nv_bfloat16>(G, q, k_cache, v_cache, positions, item_of_token, table, max_blocks, page_size,
                                           n_pages, window, scale, part_acc, part_ml, n_tok, nh, nkv, hd, chunk, n_splits,
                                           status, stream);
    else return -1;
    if (rc != 0) return rc;
    if (out == nullptr) return 0;               // the partials stay in scratch for a consumer that combines them itself
    const int threads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    if (dtype == IMPARO_DT_F32)
        launch(attn_split_combine_kernel<float>, dim3(n_tok * nh), dim3(threads), 0, stream, part_acc, part_ml, (float*)out, hd, n_splits);
    else
        launch(attn_split_combine_kernel<__nv_bfloat16>, dim3(n_tok * nh), dim3(threads), 0, stream, part_acc, part_ml, (__nv_bfloat16*)out, hd, n_splits);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// The ordered combine alone, for other kernels that produce partials in the same layout.
extern "C" int imparo_attention_split_combine(const float* part_acc, const float* part_ml, void* out, int dtype,
                                              int n_rows, int hd, int n_splits, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_splits < 1 || n_splits > COMBINE_MAX_SPLITS) return -2;
    const int threads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    if (dtype == IMPARO_DT_F32)
        launch(attn_split_combine_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, part_acc, part_ml, (float*)out, hd, n_splits);
    else if (dtype == IMPARO_DT_BF16)
        launch(attn_split_combine_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, part_acc, part_ml, (__nv_bfloat16*)out, hd, n_splits);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// ---- the variant that allocates nothing (see no_alloc.h) -----------------------------------
#include "no_alloc.h"
#include <mutex>

// The scratch of the static variant: partial accumulators, then (max, sum) pairs.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_scratch[IMPARO_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_ptr[kMaxDevices] = {};
std::mutex g_static_mutex;

// Device address of the array on the current device; resolved once per device.
int static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return IMPARO_ERR_STATIC_SCRATCH_ADDRESS;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return IMPARO_ERR_STATIC_SCRATCH_ADDRESS;
        g_static_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_static_ptr[dev];
    return 0;
}
}  // namespace

extern "C" long long imparo_paged_attention_split_static_need(int n_tok, int nh, int hd, int n_splits) {
    if (n_tok <= 0 || nh <= 0 || hd <= 0 || n_splits <= 0) return 0;
    return (long long)n_tok * nh * n_splits * (hd + 2);
}

extern "C" int imparo_paged_attention_split_static(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                                   const int* positions, const int* item_of_token,
                                                   const int* table, int max_blocks, int page_size, int n_pages,
                                                   int window, float scale, void* out,
                                                   int n_tok, int nh, int nkv, int hd, int chunk, int n_splits,
                                                   int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    // sizes first, so that the product below cannot wrap
    if (hd < 16 || hd > SPLIT_MAX_HEAD || hd % 16 != 0) return -3;
    if (nkv <= 0 || nh <= 0 || nh % nkv != 0) return -5;
    if (n_tok > 65535 || nh > 65535 || n_splits < 1 || n_splits > COMBINE_MAX_SPLITS) return -2;
    const long long need = imparo_paged_attention_split_static_need(n_tok, nh, hd, n_splits);
    if (need <= 0 || need > (long long)IMPARO_STATIC_SCRATCH_FLOATS) return IMPARO_ERR_STATIC_SCRATCH_TOO_SMALL;
    float* base = nullptr;
    const int rc = static_scratch(&base);
    if (rc != 0) return rc;
    float* part_acc = base;
    float* part_ml = base + (size_t)n_tok * nh * n_splits * hd;     // hd is a multiple of 16: stays 64-byte aligned
    return imparo_paged_attention_split(q, k_cache, v_cache, dtype, positions, item_of_token, table, max_blocks, page_size,
                                        n_pages, window, scale, out, part_acc, part_ml, n_tok, nh, nkv, hd, chunk, n_splits,
                                        status, stream);
}
