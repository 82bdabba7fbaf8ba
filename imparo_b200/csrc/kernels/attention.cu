// Attention over the paged cache: (1) per-head RMS norm + NeoX rotation of q and k and
// the write of k, v into their pages, one kernel; (2) a general attention kernel for any
// ragged batch (prompt portions beside single decoded tokens), any head size that is a
// multiple of 16 up to 256, any number of heads and groups, 32-bit or bfloat16 storage.
//
// Formulas (zeraix/imparo): per (token, head) RMS norm then rotation, before the cache
// write (imparo-model/src/cpu_support.rs:361-376); rotation pairs (i, i+n_rot/2) with
// angle = position * base^(-2i/n_rot) (imparo-cpu/src/ops.rs:551-569); cache row of a
// position = table[pos / page] * page + pos % page (imparo-cuda/native/kv_paging.cuh:25-30,
// there with 64-cell pages); scores s_j = q.k_j * scale for lo <= j <= pos, lo = 0 or
// pos+1-window, kv head = h / (heads / kv_heads), softmax with the max subtracted
// (imparo-model/src/cpu_support.rs:402-445; ops.rs:572-583).
#include "common.cuh"

namespace imparo {

constexpr int MAX_HEAD = 256;
constexpr int WARPS = 4;

// What does not depend on the previous kernel is done before the wait on it: the token's
// position, the norm weights, the rotation's sines and cosines and the cache row (the batch
// description comes from the host before the step).  After the wait: one load of the head's
// values, the norm, the rotation, the store.
// FEW: at most eight partials (or none): straight-line loads, all of a head's values in flight together
// PER: elements of a head per lane (head size up to 32 * PER), so that a head of 64 does not pay
// for the loops of a head of 256.
template <typename T, bool FEW, int PER>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_kernel(const T* __restrict__ qkv, const int* __restrict__ positions,
                          const int* __restrict__ item_of_token,
                          const float* __restrict__ q_w, const float* __restrict__ k_w,
                          const float* __restrict__ inv_freq, int n_rot, float eps,
                          T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                          const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                          int nh, int nkv, int hd, const float* __restrict__ part, int parts, size_t part_stride,
                          int* status) {
    __shared__ float rowbuf[WARPS][MAX_HEAD];
    constexpr int PAIRS = (PER + 1) / 2;
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hh = blockIdx.y * WARPS + warp;
    const int total = nh + 2 * nkv;
    if (hh >= total) return;
    const int in_width = total * hd;
    const T* src = qkv + (size_t)t * in_width + (size_t)hh * hd;
    float* row = rowbuf[warp];
    const int pos = positions[t];
    const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
    const int half = n_rot >> 1;

    float wreg[PER], sn[PAIRS], cs[PAIRS];
    if (is_q || is_k) {
        const float* w = is_q ? q_w : k_w;                  // null: this side has no per-head norm
#pragma unroll
        for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; wreg[j] = d < hd ? (w ? w[d] : 1.f) : 0.f; }
        if (inv_freq) {
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int i = lane + 32 * j;
                sn[j] = 0.f; cs[j] = 1.f;
                if (i < half) sincosf((float)pos * inv_freq[i], &sn[j], &cs[j]);
            }
        }
    }
    T* dst = nullptr;
    int bad_page = 0;
    if (is_q) {
        dst = q_out + (size_t)t * nh * hd + (size_t)hh * hd;
    } else {
        const int kvh = is_k ? hh - nh : hh - nh - nkv;
        const int blk = pos / page_size;
        int page = -1;
        if (blk < max_blocks) page = table[(size_t)item_of_token[t] * max_blocks + blk];
        if (page < 0 || page >= n_pages) {
            bad_page = page;                                 // reported after the wait
        } else {
            const size_t r = (size_t)page * page_size + (pos % page_size);
            dst = (is_k ? k_cache : v_cache) + r * ((size_t)nkv * hd) + (size_t)kvh * hd;
        }
    }
    pdl_wait();
    if (dst == nullptr) {
        if (lane == 0) report(status, IMPARO_ST_PAGE_RANGE, 2, t, bad_page);
        return;
    }

    float val[PER];
    float ss = 0.f;
    if (parts > 0) {
        // the product before this kernel was cut along K and left its partial results
        // [parts][tokens][width]: summed here in split order and rounded as a stored tensor would be
        const float* ps = part + (size_t)t * in_width + (size_t)hh * hd;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int d = lane + 32 * j;
            float acc = 0.f;
            if (d < hd) {
                if (FEW) {
                    float v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = u < parts ? __ldcg(ps + (size_t)u * part_stride + d) : 0.f;
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (u < parts) acc += v[u];
                } else {
                    for (int s0 = 0; s0 < parts; s0 += 8) {
                        float v[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) v[u] = s0 + u < parts ? __ldcg(ps + (size_t)(s0 + u) * part_stride + d) : 0.f;
#pragma unroll
                        for (int u = 0; u < 8; ++u) if (s0 + u < parts) acc += v[u];
                    }
                }
            }
            val[j] = to_f32(from_f32<T>(acc));
            ss += val[j] * val[j];
        }
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int d = lane + 32 * j;
            val[j] = d < hd ? to_f32(src[d]) : 0.f;
            ss += val[j] * val[j];
        }
    }
    if (is_q || is_k) {
        ss = warp_sum(ss);
        const float scale = (is_q ? q_w : k_w) ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; if (d < hd) row[d] = val[j] * scale * wreg[j]; }
        __syncwarp();
        if (inv_freq) {
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int i = lane + 32 * j;
                if (i < half) {
                    const float x0 = row[i], x1 = row[i + half];
                    row[i] = x0 * cs[j] - x1 * sn[j];
                    row[i + half] = x0 * sn[j] + x1 * cs[j];
                }
            }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; if (d < hd) dst[d] = from_f32<T>(row[d]); }
    } else {
#pragma unroll
        for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; if (d < hd) dst[d] = from_f32<T>(val[j]); }
    }
}

// Many tokens (a prompt portion), stored input, and a rotation whose pairs (i, i + n_rot/2) fall
// into the same lane (n_rot/2 a multiple of 32, e.g. heads of 64 or 128 fully rotated): a block owns
// one token, its four warps share the token's heads, the sines and cosines of the position are
// computed once per warp instead of once per head, and norm and rotation stay in registers.
template <typename T, int PER>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_rows_kernel(const T* __restrict__ qkv, const int* __restrict__ positions,
                         const int* __restrict__ item_of_token,
                         const float* __restrict__ q_w, const float* __restrict__ k_w,
                         const float* __restrict__ inv_freq, int n_rot, float eps,
                         T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                         const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                         int nh, int nkv, int hd, int* status) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total = nh + 2 * nkv;
    const int pos = positions[t];
    const int hj = n_rot >> 6;                               // register distance of a rotation pair: (n_rot / 2) / 32
    float wq[PER], wk[PER], sn[PER], cs[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int d = lane + 32 * j;
        wq[j] = d < hd ? (q_w ? q_w[d] : 1.f) : 0.f;         // null weights: no per-head norm on that side
        wk[j] = (d < hd && nkv > 0) ? (k_w ? k_w[d] : 1.f) : 0.f;
        sn[j] = 0.f; cs[j] = 1.f;
        if (inv_freq && j < hj) sincosf((float)pos * inv_freq[d], &sn[j], &cs[j]);
    }
    size_t cache_row = 0;
    int page = 0;
    if (nkv > 0) {
        const int blk = pos / page_size;
        page = blk < max_blocks ? table[(size_t)item_of_token[t] * max_blocks + blk] : -1;
        if (page >= 0 && page < n_pages) cache_row = (size_t)page * page_size + (pos % page_size);
    }
    pdl_wait();
    const T* src = qkv + (size_t)t * total * hd;
    float nxt[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; nxt[j] = (warp < total && d < hd) ? to_f32(src[(size_t)warp * hd + d]) : 0.f; }
    for (int hh = warp; hh < total; hh += WARPS) {
        float val[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) val[j] = nxt[j];
        if (hh + WARPS < total) {                            // the next head's values are on their way meanwhile
#pragma unroll
            for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; nxt[j] = d < hd ? to_f32(src[(size_t)(hh + WARPS) * hd + d]) : 0.f; }
        }
        const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
        T* dst;
        if (is_q) {
            dst = q_out + (size_t)t * nh * hd + (size_t)hh * hd;
        } else {
            if (page < 0 || page >= n_pages) {
                if (lane == 0) report(status, IMPARO_ST_PAGE_RANGE, 2, t, page);
                return;
            }
            const int kvh = is_k ? hh - nh : hh - nh - nkv;
            dst = (is_k ? k_cache : v_cache) + cache_row * ((size_t)nkv * hd) + (size_t)kvh * hd;
        }
        if (is_q || is_k) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < PER; ++j) ss += val[j] * val[j];
            ss = warp_sum(ss);
            const float scale = (is_q ? q_w : k_w) ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.0f;
#pragma unroll
            for (int j = 0; j < PER; ++j) val[j] = val[j] * scale * (is_q ? wq[j] : wk[j]);
            if (inv_freq) {
#pragma unroll
                for (int j = 0; j < PER / 2; ++j) {
                    if (j < hj) {
                        // the pair (lane + 32 j, lane + 32 j + n_rot/2): registers j and j + hj
                        float x0 = val[j], x1 = 0.f;
#pragma unroll
                        for (int q = 0; q < PER; ++q) if (q == j + hj) x1 = val[q];
                        const float r0 = x0 * cs[j] - x1 * sn[j], r1 = x0 * sn[j] + x1 * cs[j];
                        val[j] = r0;
#pragma unroll
                        for (int q = 0; q < PER; ++q) if (q == j + hj) val[q] = r1;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; if (d < hd) dst[d] = from_f32<T>(val[j]); }
    }
}

// bfloat16, many tokens, a head fully rotated (n_rot == head size) or not at all, head size 32 * V: a lane owns V
// consecutive dims of a head (one load of 2 V bytes), so the lower half of a head lies in lanes 0-15 and the pair
// (i, i + head/2) of the rotation in lanes l and l ^ 16: one shuffle per value.  A block owns one token, its eight warps
// share the token's heads, FOUR heads at a time per warp with all their loads in flight together; sines and cosines
// of the position once per warp.  The kernel above keeps one head in flight per warp and is bound by that.
template <int V>
__global__ void __launch_bounds__(256)
qk_norm_rope_rows_vec_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                             const int* __restrict__ item_of_token,
                             const float* __restrict__ q_w, const float* __restrict__ k_w,
                             const float* __restrict__ inv_freq, float eps,
                             __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                             __nv_bfloat16* __restrict__ v_cache,
                             const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                             int nh, int nkv, int* status) {
    constexpr int HD = 32 * V, NW = 8, BATCH = 4;
    struct alignas(2 * V) Vec { __nv_bfloat16 e[V]; };
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total = nh + 2 * nkv;
    const int pos = positions[t];
    // the position's sines and cosines: computed once per block (the first threads, one frequency each) and shared;
    // eight warps computing them each would spend nearly half of the kernel's instructions on them
    __shared__ float sn_s[HD / 2], cs_s[HD / 2];
    if (inv_freq && threadIdx.x < HD / 2) sincosf((float)pos * inv_freq[threadIdx.x], &sn_s[threadIdx.x], &cs_s[threadIdx.x]);
    float wq[V], wk[V], sn[V], cs[V];
#pragma unroll
    for (int e = 0; e < V; ++e) {
        const int d = V * lane + e;
        wq[e] = q_w ? q_w[d] : 1.f;                          // null weights: no per-head norm on that side
        wk[e] = (k_w && nkv > 0) ? k_w[d] : 1.f;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < V; ++e) {
        const int d = V * lane + e;
        sn[e] = inv_freq ? sn_s[d % (HD / 2)] : 0.f;
        cs[e] = inv_freq ? cs_s[d % (HD / 2)] : 1.f;
    }
    size_t cache_row = 0;
    int page = 0;
    if (nkv > 0) {
        const int blk = pos / page_size;
        page = blk < max_blocks ? table[(size_t)item_of_token[t] * max_blocks + blk] : -1;
        if (page >= 0 && page < n_pages) cache_row = (size_t)page * page_size + (pos % page_size);
    }
    pdl_wait();
    if (nkv > 0 && (page < 0 || page >= n_pages) && threadIdx.x == 0)
        report(status, IMPARO_ST_PAGE_RANGE, 2, t, page);     // the token's keys and values are skipped below, its queries written
    const __nv_bfloat16* src = qkv + (size_t)t * total * HD + V * lane;
    const bool upper = lane >= 16;
    for (int h0 = warp * BATCH; h0 < total; h0 += NW * BATCH) {
        Vec in[BATCH];
#pragma unroll
        for (int u = 0; u < BATCH; ++u)
            if (h0 + u < total) in[u] = *reinterpret_cast<const Vec*>(src + (size_t)(h0 + u) * HD);
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            const int hh = h0 + u;
            if (hh >= total) break;
            const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
            float val[V];
#pragma unroll
            for (int e = 0; e < V; ++e) val[e] = __bfloat162float(in[u].e[e]);
            if (is_q || is_k) {
                const float* wn = is_q ? q_w : k_w;
                float scale = 1.f;
                if (wn) {
                    float ss = 0.f;
#pragma unroll
                    for (int e = 0; e < V; ++e) ss += val[e] * val[e];
                    ss = warp_sum(ss);
                    scale = 1.0f / sqrtf(ss / (float)HD + eps);
                }
#pragma unroll
                for (int e = 0; e < V; ++e) val[e] = val[e] * scale * (is_q ? wq[e] : wk[e]);
                if (inv_freq) {
#pragma unroll
                    for (int e = 0; e < V; ++e) {
                        const float other = __shfl_xor_sync(0xffffffffu, val[e], 16);
                        // lower half: x0 cos - x1 sin with x1 = other; upper half: x0 sin + x1 cos with x0 = other
                        val[e] = upper ? other * sn[e] + val[e] * cs[e] : val[e] * cs[e] - other * sn[e];
                    }
                }
            }
            __nv_bfloat16* dst;
            if (is_q) {
                dst = q_out + ((size_t)t * nh + hh) * HD;
            } else {
                if (page < 0 || page >= n_pages) continue;
                const int kvh = is_k ? hh - nh : hh - nh - nkv;
                dst = (is_k ? k_cache : v_cache) + cache_row * ((size_t)nkv * HD) + (size_t)kvh * HD;
            }
            Vec o;
#pragma unroll
            for (int e = 0; e < V; ++e) o.e[e] = __float2bfloat16_rn(val[e]);
            *reinterpret_cast<Vec*>(dst + V * lane) = o;
        }
    }
}

// The same for heads of 64 or 128 with a WARP per token: a lane owns 8 consecutive dims of a head (16-byte loads and
// stores), HD / 8 lanes make a head, so one load instruction of the warp fetches 4 (or 2) heads, and all of a token's heads
// are in flight before the first is used.  The kernel above gives a token a block of eight warps: its chain of
// dependent reads (position, table, the values) is paid per block with four to eight blocks on an SM, 20 us for 2,048
// tokens of 48 heads; here 64 tokens are in flight per SM.  Rotation pairs (i, i + HD/2) lie HD/16 lanes apart.
template <int HD>
__global__ void __launch_bounds__(128)
qk_norm_rope_token_warp_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                               const int* __restrict__ item_of_token,
                               const float* __restrict__ q_w, const float* __restrict__ k_w,
                               const float* __restrict__ inv_freq, float eps,
                               __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                               __nv_bfloat16* __restrict__ v_cache,
                               const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                               int n_tok, int nh, int nkv, int share, int* status) {
    constexpr int LPH = HD / 8, HPL = 32 / LPH, CHUNK = 8, NF = HD / 64;      // lanes per head, heads per load, loads in flight, frequencies per lane
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    // share: warps that divide a token's heads between them.  A portion of a few hundred tokens is fewer warps than the
    // SMs have schedulers, each walking its token's heads in rounds of dependent loads: 6.5 us for 512 tokens of 40
    // heads; shared out, every warp has one round.
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int t = w / share, mine = w - t * share;
    if (t >= n_tok) return;
    const int total = nh + 2 * nkv;
    const int sub = lane % LPH, hsel = lane / LPH;           // which 8 dims of the head, which head of the load
    const int pos = positions[t];
    int page = 0;
    size_t cache_row = 0;
    if (nkv > 0) {
        const int blk = pos / page_size;
        page = blk < max_blocks ? table[(size_t)item_of_token[t] * max_blocks + blk] : -1;
        if (page >= 0 && page < n_pages) cache_row = (size_t)page * page_size + (pos % page_size);
    }
    float wq[8], wk[8], sn[8], cs[8];
    {
        const float4* q4 = reinterpret_cast<const float4*>(q_w ? q_w + 8 * sub : nullptr);
        const float4* k4 = reinterpret_cast<const float4*>((k_w && nkv > 0) ? k_w + 8 * sub : nullptr);
        const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 a = q4 ? q4[0] : one, b = q4 ? q4[1] : one, c = k4 ? k4[0] : one, d = k4 ? k4[1] : one;
        wq[0] = a.x; wq[1] = a.y; wq[2] = a.z; wq[3] = a.w; wq[4] = b.x; wq[5] = b.y; wq[6] = b.z; wq[7] = b.w;
        wk[0] = c.x; wk[1] = c.y; wk[2] = c.z; wk[3] = c.w; wk[4] = d.x; wk[5] = d.y; wk[6] = d.z; wk[7] = d.w;
    }
    // the position's HD / 2 sines and cosines: NF per lane, then each lane fetches those of its 8 dims
    {
        float s_own[NF], c_own[NF];
#pragma unroll
        for (int f = 0; f < NF; ++f) {
            s_own[f] = 0.f; c_own[f] = 1.f;
            if (inv_freq) sincosf((float)pos * inv_freq[lane + 32 * f], &s_own[f], &c_own[f]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int i = (8 * sub + e) % (HD / 2);          // the pair's index
            float sv = __shfl_sync(0xffffffffu, s_own[0], i & 31), cv = __shfl_sync(0xffffffffu, c_own[0], i & 31);
            if (NF > 1) {
                const float s1 = __shfl_sync(0xffffffffu, s_own[NF - 1], i & 31), c1 = __shfl_sync(0xffffffffu, c_own[NF - 1], i & 31);
                if (i >= 32) { sv = s1; cv = c1; }
            }
            sn[e] = sv; cs[e] = cv;
        }
    }
    pdl_wait();
    if (nkv > 0 && (page < 0 || page >= n_pages) && lane == 0)
        report(status, IMPARO_ST_PAGE_RANGE, 2, t, page);     // the token's keys and values are skipped below, its queries written
    const __nv_bfloat16* src = qkv + (size_t)t * total * HD + 8 * sub;
    const bool upper = sub >= LPH / 2;
    const int all_loads = (total + HPL - 1) / HPL;
    const int per_warp = (all_loads + share - 1) / share;
    const int n_loads = min(all_loads, (mine + 1) * per_warp);
    for (int g0 = mine * per_warp; g0 < n_loads; g0 += CHUNK) {
        uint4 in[CHUNK];
#pragma unroll
        for (int u = 0; u < CHUNK; ++u) {
            const int hh = (g0 + u) * HPL + hsel;
            if (g0 + u < n_loads && hh < total) in[u] = *reinterpret_cast<const uint4*>(src + (size_t)hh * HD);
        }
#pragma unroll
        for (int u = 0; u < CHUNK; ++u) {
            const int hh = (g0 + u) * HPL + hsel;
            const bool live = g0 + u < n_loads && hh < total;          // (the shuffles below are executed by every lane)
            if (g0 + u >= n_loads) break;
            const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
            float val[8];
            {
                const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&in[u]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = live ? __bfloat1622float2(p2[e]) : make_float2(0.f, 0.f);
                    val[2 * e] = f.x; val[2 * e + 1] = f.y;
                }
            }
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += val[e] * val[e];
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const bool normed = (is_q && q_w) || (is_k && k_w);
            const float scale = normed ? 1.0f / sqrtf(ss / (float)HD + eps) : 1.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float v = val[e];
                if (is_q || is_k) v = v * scale * (is_q ? wq[e] : wk[e]);
                const float other = __shfl_xor_sync(0xffffffffu, v, LPH / 2);
                if ((is_q || is_k) && inv_freq)
                    v = upper ? other * sn[e] + v * cs[e] : v * cs[e] - other * sn[e];
                val[e] = v;
            }
            if (!live) continue;
            __nv_bfloat16* dst;
            if (is_q) {
                dst = q_out + ((size_t)t * nh + hh) * HD;
            } else {
                if (page < 0 || page >= n_pages) continue;
                const int kvh = is_k ? hh - nh : hh - nh - nkv;
                dst = (is_k ? k_cache : v_cache) + cache_row * ((size_t)nkv * HD) + (size_t)kvh * HD;
            }
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(val[2 * e], val[2 * e + 1]);
            *reinterpret_cast<uint4*>(dst + 8 * sub) = o;
        }
    }
}

// ---- general paged attention ---------------------------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> { using type = float4; static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { using type = uint4; static constexpr int N = 8; };

__device__ __forceinline__ float dot_vec(const float4& k, const float* q) {
    return k.x * q[0] + k.y * q[1] + k.z * q[2] + k.w * q[3];
}
__device__ __forceinline__ float dot_vec(const uint4& k, const float* q) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&k);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        s += f.x * q[2 * i] + f.y * q[2 * i + 1];
    }
    return s;
}

// One warp per (token, head).  Keys are walked 32 at a time in position order: each lane
// scores one key, the warp folds the chunk into the running max / sum, then all lanes
// accumulate the chunk's values, each lane owning head dimensions lane, lane+32, ...
// The walk depends only on (position, window): never on the batch around the token.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int* __restrict__ positions, const int* __restrict__ item_of_token,
                       const int* __restrict__ table, int max_blocks, int page_size, int n_pages,
                       int window, float scale, T* __restrict__ out, int nh, int nkv, int hd, int* status) {
    __shared__ __align__(16) float qbuf[WARPS][MAX_HEAD];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= nh) return;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    const int* tab = table + (size_t)item_of_token[t] * max_blocks;
    const size_t kvw = (size_t)nkv * hd;
    float* qs = qbuf[warp];
    const T* qrow = q + ((size_t)t * nh + h) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();

    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    constexpr int PER = MAX_HEAD / 32;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    using V = typename Vec<T>::type;
    constexpr int VN = Vec<T>::N;

    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        float s = -INFINITY;
        int rowi = -1;
        if (j <= pos) {
            const int blk = j / page_size;
            const int page = blk < max_blocks ? tab[blk] : -1;
            if (page < 0 || page >= n_pages) {
                report(status, IMPARO_ST_PAGE_RANGE, 3, t, page);
            } else {
                rowi = page * page_size + (j % page_size);
                const V* kp = reinterpret_cast<const V*>(k_cache + (size_t)rowi * kvw + (size_t)kvh * hd);
                float d = 0.f;
                for (int c = 0; c < hd / VN; ++c) d += dot_vec(kp[c], qs + c * VN);
                s = d * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;   // a chunk of unreadable keys only (already reported)
        const float p = (rowi >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] *= corr;
        m = m_new;
        const int cnt = min(32, pos - base + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int rj = __shfl_sync(0xffffffffu, rowi, jj);
            if (rj < 0) continue;
            const T* vp = v_cache + (size_t)rj * kvw + (size_t)kvh * hd;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] += pj * to_f32(vp[d]);
            }
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* orow = out + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace imparo

using namespace imparo;

// qkv: [n_tok, (nh + 2 nkv) * hd] of the dtype; or, when parts > 0, float partial results
// [parts][n_tok][width] (split s at qkv + s * part_stride floats) of a product cut along K.
extern "C" int imparo_qk_norm_rope_store(const void* qkv, int dtype, const int* positions, const int* item_of_token,
                                         const float* q_w, const float* k_w, const float* inv_freq, int n_rot, float eps,
                                         void* q_out, void* k_cache, void* v_cache,
                                         const int* table, int max_blocks, int page_size, int n_pages,
                                         int n_tok, int nh, int nkv, int hd, int parts, long long part_stride,
                                         int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd < 16 || hd > MAX_HEAD || hd % 16 != 0) return -3;
    if (n_rot < 0 || n_rot > hd || (n_rot & 1)) return -4;
    if (parts < 0 || (parts > 0 && part_stride < (long long)n_tok * (nh + 2 * nkv) * hd)) return -2;
    dim3 grid(n_tok, (nh + 2 * nkv + WARPS - 1) / WARPS);
    const float* part = parts > 0 ? (const float*)qkv : nullptr;
    if (n_tok >= 256 && parts == 0 && dtype == IMPARO_DT_BF16 && (hd == 64 || hd == 128 || hd == 256) &&
        (inv_freq == nullptr || n_rot == hd) &&
        (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0) {
        // a prompt portion in bfloat16 with whole-head rotation: vector loads, four heads in flight per warp
#define IMPARO_QKV(V_) launch(qk_norm_rope_rows_vec_kernel<V_>, dim3(n_tok), dim3(256), 0, stream, (const __nv_bfloat16*)qkv, positions, \
            item_of_token, q_w, k_w, inv_freq, eps, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, table, \
            max_blocks, page_size, n_pages, nh, nkv, status)
        // warps per token: enough to give the device about 2,048 warps, at most 8 (and no more than the token has loads)
        int share = n_tok >= 2048 ? 1 : n_tok >= 1024 ? 2 : n_tok >= 512 ? 4 : 8;
        {
            const int loads = (nh + 2 * nkv + (hd == 64 ? 4 : 2) - 1) / (hd == 64 ? 4 : 2);
            while (share > 1 && share > loads) share >>= 1;
        }
#define IMPARO_QKW(HD_) launch(qk_norm_rope_token_warp_kernel<HD_>, dim3((unsigned)(((long long)n_tok * share + 3) / 4)), dim3(128), 0, stream, (const __nv_bfloat16*)qkv, \
            positions, item_of_token, q_w, k_w, inv_freq, eps, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, table, \
            max_blocks, page_size, n_pages, n_tok, nh, nkv, share, status)
        const bool w_ok = (((uintptr_t)q_w | (uintptr_t)k_w) & 15) == 0;                  // the norm weights are read 16 bytes at a time
        if (hd == 64 && w_ok) IMPARO_QKW(64); else if (hd == 128 && w_ok) IMPARO_QKW(128);
        else if (hd == 64) IMPARO_QKV(2); else if (hd == 128) IMPARO_QKV(4); else IMPARO_QKV(8);
#undef IMPARO_QKW
#undef IMPARO_QKV
        IMPARO_CHECK_LAUNCH();
        return 0;
    }
    if (n_tok >= 256 && parts == 0 && hd % 32 == 0 && hd <= 128 && (inv_freq == nullptr || (n_rot >= 64 && n_rot % 64 == 0))) {
        // a prompt portion: the register-only kernel, one block per token
#define IMPARO_QKR(T_, PER_) launch(qk_norm_rope_rows_kernel<T_, PER_>, dim3(n_tok), dim3(WARPS * 32), 0, stream, (const T_*)qkv, \
            positions, item_of_token, q_w, k_w, inv_freq, n_rot, eps, (T_*)q_out, (T_*)k_cache, (T_*)v_cache, table, max_blocks, \
            page_size, n_pages, nh, nkv, hd, status)
        if (dtype == IMPARO_DT_F32) { if (hd <= 64) IMPARO_QKR(float, 2); else IMPARO_QKR(float, 4); }
        else if (dtype == IMPARO_DT_BF16) { if (hd <= 64) IMPARO_QKR(__nv_bfloat16, 2); else IMPARO_QKR(__nv_bfloat16, 4); }
        else return -1;
#undef IMPARO_QKR
        IMPARO_CHECK_LAUNCH();
        return 0;
    }
#define IMPARO_QK3(T_, FEW_, PER_) launch(qk_norm_rope_store_kernel<T_, FEW_, PER_>, grid, dim3(WARPS * 32), 0, stream, \
            (const T_*)qkv, positions, item_of_token, q_w, k_w, inv_freq, n_rot, eps, (T_*)q_out, (T_*)k_cache, (T_*)v_cache, \
            table, max_blocks, page_size, n_pages, nh, nkv, hd, part, parts, (size_t)part_stride, status)
#define IMPARO_QK(T_, FEW_) do { if (hd <= 64) IMPARO_QK3(T_, FEW_, 2); else if (hd <= 128) IMPARO_QK3(T_, FEW_, 4); \
                                 else IMPARO_QK3(T_, FEW_, 8); } while (0)
    if (dtype == IMPARO_DT_F32) {
        if (parts <= 8) IMPARO_QK(float, true); else IMPARO_QK(float, false);
    } else if (dtype == IMPARO_DT_BF16) {
        if (parts <= 8) IMPARO_QK(__nv_bfloat16, true); else IMPARO_QK(__nv_bfloat16, false);
    }
#undef IMPARO_QK3
#undef IMPARO_QK
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_paged_attention(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                      const int* positions, const int* item_of_token,
                                      const int* table, int max_blocks, int page_size, int n_pages,
                                      int window, float scale, void* out,
                                      int n_tok, int nh, int nkv, int hd, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (hd < 16 || hd > MAX_HEAD || hd % 16 != 0) return -3;
    if (nkv <= 0 || nh % nkv != 0) return -5;
    dim3 grid(n_tok, (nh + WARPS - 1) / WARPS);
    if (dtype == IMPARO_DT_F32)
        launch(paged_attention_kernel<float>, grid, dim3(WARPS * 32), 0, stream,
            (const float*)q, (const float*)k_cache, (const float*)v_cache, positions, item_of_token, table,
            max_blocks, page_size, n_pages, window, scale, (float*)out, nh, nkv, hd, status);
    else if (dtype == IMPARO_DT_BF16)
        launch(paged_attention_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), 0, stream,
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions,
            item_of_token, table, max_blocks, page_size, n_pages, window, scale, (__nv_bfloat16*)out, nh, nkv, hd, status);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}
