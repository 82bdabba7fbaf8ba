// Attention for prompt portions over the paged cache on tensor cores (bfloat16, head size
// 64 or 128): a CTA owns up to 64 query rows = (64 / G) consecutive tokens of ONE request
// times the G query heads that share a kv head, walks the keys 64 at a time in position
// order, scores with mma.sync m16n8k16 (bfloat16 in, 32-bit out), keeps the running max and
// sum per row in 32-bit, and accumulates P*V with the same instruction.  Keys and values of a
// block are read once for the whole group.  The reference's prefill kernel has the same
// shape for its f16 cache (imparo-cuda/native/sm80/attention_prefill_mma_d64_f16.cuh:29:
// "CTA = 16 query tokens x 4 GQA heads x 1 KV head, walks 64-key updates in order").
//
// Formulas: scores q.k * scale for lo <= key <= position, lo = 0 or position+1-window, no
// mask tensor, softmax with the max subtracted (imparo-model/src/cpu_support.rs:402-445).
// Which tokens form a tile is derived on the device from the batch's row starts, so a tile
// never holds rows of two requests; a token's result does not depend on its neighbours in
// the tile (every row has its own max, sum and mask).
#include "common.cuh"

namespace imparo {
namespace pf {

constexpr int ROWS = 64;          // query rows per CTA
constexpr int KEYS = 64;          // keys per step
constexpr int THREADS = 128;      // 4 warps x 16 rows

// 2^x by the hardware's approximation (2 ulp; inputs at or below -126 give 0, -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                 // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of 16-byte chunk c of row r in a [rows][HD] bfloat16 tile, XOR-swizzled so that
// the eight rows an ldmatrix reads fall into distinct banks
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)r * (HD * 2) + (uint32_t)((c ^ (r & 7)) << 4); }

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ item_row_start,
                    const int* __restrict__ item_start_pos, int n_items, const int* __restrict__ table, int max_blocks,
                    int page_size, int n_pages, int window, float scale, __nv_bfloat16* __restrict__ out,
                    int nh, int nkv, int* status) {
    constexpr int CH = HD / 8;                    // 16-byte chunks per row
    constexpr int KT = HD / 16;                   // k-steps of the score product
    constexpr int NT_O = HD / 8;                  // n-tiles of the output
    extern __shared__ __align__(128) uint8_t pf_smem[];
    uint8_t* q_s = pf_smem;
    uint8_t* k_s[2] = {q_s + ROWS * HD * 2, q_s + ROWS * HD * 2 + KEYS * HD * 2};
    uint8_t* v_s[2] = {k_s[1] + KEYS * HD * 2, k_s[1] + 2 * KEYS * HD * 2};
    pdl_trigger();

    const int G = nh / nkv;
    const int TQ = ROWS / G;                      // tokens per tile
    const int kvh = blockIdx.y;
    // which request and which of its tokens: tiles are numbered request by request
    int item = 0, tile = blockIdx.x, n_item = 0, row0 = 0;
    for (; item < n_items; ++item) {
        row0 = item_row_start[item];
        n_item = item_row_start[item + 1] - row0;
        const int tiles = (n_item + TQ - 1) / TQ;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (item >= n_items) return;
    const int tok0 = tile * TQ;                               // first token of the tile within its request's portion
    const int n_tok = min(TQ, n_item - tok0);
    const int n_rows = n_tok * G;
    const int pos0 = item_start_pos[item] + tok0;             // position of the tile's first token
    const int pos_last = pos0 + n_tok - 1;
    const int* tab = table + (size_t)item * max_blocks;
    const size_t kvw = (size_t)nkv * HD;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tg = lane & 3;

    pdl_wait();          // up to here only the batch description was read, which the host wrote before the step

    // ---- queries -> shared memory (row r = token r / G, head kvh*G + r % G) ----
    for (int i = tid; i < ROWS * CH; i += THREADS) {
        const int r = i / CH, c = i % CH;
        const bool valid = r < n_rows;
        const size_t t = (size_t)row0 + tok0 + (valid ? r / G : 0);
        const __nv_bfloat16* src = q + (t * nh + (size_t)kvh * G + (valid ? r % G : 0)) * HD + c * 8;
        cp_async16(q_s + tile_off<HD>(r, c), src, valid);
    }
    cp_commit();

    const int lo_min = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int kb_first = lo_min / KEYS, kb_last = pos_last / KEYS;

    auto load_kv = [&](int kb, int buf) {
        for (int i = tid; i < KEYS * CH; i += THREADS) {
            const int r = i / CH, c = i % CH;
            const int j = kb * KEYS + r;
            bool valid = j <= pos_last && j >= lo_min;
            size_t rowi = 0;
            if (valid) {
                const int blk = j / page_size;
                const int page = blk < max_blocks ? tab[blk] : -1;
                if (page < 0 || page >= n_pages) {
                    if (c == 0) report(status, IMPARO_ST_PAGE_RANGE, 6, item, page);
                    valid = false;
                } else {
                    rowi = (size_t)page * page_size + (j % page_size);
                }
            }
            const size_t off = rowi * kvw + (size_t)kvh * HD + c * 8;
            cp_async16(k_s[buf] + tile_off<HD>(r, c), k_cache + off, valid);
            cp_async16(v_s[buf] + tile_off<HD>(r, c), v_cache + off, valid);
        }
        cp_commit();
    };
    load_kv(kb_first, 0);

    // ---- this warp's query fragments ----
    cp_wait<1>();
    __syncthreads();
    uint32_t qf[KT][4];
    {
        const int m = lane >> 3, rin = lane & 7;
        const int r = warp * 16 + (m & 1) * 8 + rin;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) ldmatrix4(qf[kt], smem_addr(q_s + tile_off<HD>(r, kt * 2 + (m >> 1))));
    }
    // rows of this thread: warp*16 + g and + 8; their positions and window starts
    const int r_a = warp * 16 + g, r_b = r_a + 8;
    const int pos_a = pos0 + r_a / G, pos_b = pos0 + r_b / G;
    const int lo_a = (window > 0 && pos_a + 1 > window) ? pos_a + 1 - window : 0;
    const int lo_b = (window > 0 && pos_b + 1 > window) ? pos_b + 1 - window : 0;

    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const float sl2 = scale * 1.4426950408889634f;            // scores in units of log2(e)

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int buf = (kb - kb_first) & 1;
        if (kb < kb_last) load_kv(kb + 1, buf ^ 1);
        if (kb < kb_last) cp_wait<1>(); else cp_wait<0>();
        __syncthreads();

        // ---- scores: 16 rows x 64 keys per warp ----
        float s[KEYS / 8][4];
#pragma unroll
        for (int n = 0; n < KEYS / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        {
            const int m = lane >> 3, rin = lane & 7;
#pragma unroll
            for (int np = 0; np < KEYS / 16; ++np) {                 // pairs of 8-key tiles
                const int key = np * 16 + (m >> 1) * 8 + rin;
#pragma unroll
                for (int kt = 0; kt < KT; ++kt) {
                    uint32_t b[4];
                    ldmatrix4(b, smem_addr(k_s[buf] + tile_off<HD>(key, kt * 2 + (m & 1))));
                    mma16816(s[2 * np], qf[kt], b[0], b[1]);
                    mma16816(s[2 * np + 1], qf[kt], b[2], b[3]);
                }
            }
        }
        // ---- mask by position, running max and sum ----
        const int key0 = kb * KEYS + 2 * tg;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = key0 + n * 8 + e;
                const bool ok_a = j <= pos_a && j >= lo_a, ok_b = j <= pos_b && j >= lo_b;
                s[n][e] = ok_a ? s[n][e] * sl2 : -INFINITY;
                s[n][2 + e] = ok_b ? s[n][2 + e] * sl2 : -INFINITY;
                mx_a = fmaxf(mx_a, s[n][e]);
                mx_b = fmaxf(mx_b, s[n][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ca = (m_a == -INFINITY) ? 0.f : exp2f(m_a - mn_a);
        const float cb = (m_b == -INFINITY) ? 0.f : exp2f(m_b - mn_b);
        const float ba = (mn_a == -INFINITY) ? 0.f : mn_a, bb = (mn_b == -INFINITY) ? 0.f : mn_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int n = 0; n < KEYS / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[n][e] = exp2f(s[n][e] - ba);               // exp2(-inf) = 0 for masked keys
                s[n][2 + e] = exp2f(s[n][2 + e] - bb);
                sum_a += s[n][e];
                sum_b += s[n][2 + e];
            }
        }
        l_a = l_a * ca + sum_a;                               // per-thread partial sums; folded across the quad at the end
        l_b = l_b * cb + sum_b;
        m_a = mn_a;
        m_b = mn_b;
#pragma unroll
        for (int n = 0; n < NT_O; ++n) { o[n][0] *= ca; o[n][1] *= ca; o[n][2] *= cb; o[n][3] *= cb; }

        // ---- O += P * V ----
        {
            const int m = lane >> 3, rin = lane & 7;
#pragma unroll
            for (int kt = 0; kt < KEYS / 16; ++kt) {                 // 16 keys per step
                uint32_t a[4];
                a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
                a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
                a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
                a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
                const int key = kt * 16 + (m & 1) * 8 + rin;
#pragma unroll
                for (int np = 0; np < NT_O / 2; ++np) {               // pairs of 8-dim tiles
                    uint32_t b[4];
                    ldmatrix4_trans(b, smem_addr(v_s[buf] + tile_off<HD>(key, np * 2 + (m >> 1))));
                    mma16816(o[2 * np], a, b[0], b[1]);
                    mma16816(o[2 * np + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                       // the buffer is refilled two steps on
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float ia = l_a > 0.f ? 1.0f / l_a : 0.f, ib = l_b > 0.f ? 1.0f / l_b : 0.f;
    // ---- write out[token, head, dim] ----
    if (r_a < n_rows) {
        __nv_bfloat16* dst = out + (((size_t)row0 + tok0 + r_a / G) * nh + (size_t)kvh * G + r_a % G) * HD;
#pragma unroll
        for (int n = 0; n < NT_O; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * tg) = pack_bf16(o[n][0] * ia, o[n][1] * ia);
    }
    if (r_b < n_rows) {
        __nv_bfloat16* dst = out + (((size_t)row0 + tok0 + r_b / G) * nh + (size_t)kvh * G + r_b % G) * HD;
#pragma unroll
        for (int n = 0; n < NT_O; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * tg) = pack_bf16(o[n][2] * ib, o[n][3] * ib);
    }
}


// ---- single query tokens (decode rows), split over key chunks, on tensor cores -----------
// One CTA per (key chunk, kv head, token).  The token's G query heads are rows 0..G-1 of a
// 16-row MMA tile (the rest is padding) and are read straight into registers.  The chunk's keys
// are staged 64 at a time with cp.async (double buffer); each of the four warps scores 16 of the
// 64 keys, keeps its own running max / sum / accumulator, and the warps are folded in warp order
// at the end.  The result is an unnormalised partial per (token, head, chunk) for the ordered
// combine kernel of attention_split.cu (same scratch layout: part_acc [T, nh, S, HD], part_ml
// [T, nh, S, 2]).  Tiles of keys that earlier steps wrote are requested before the wait on the
// previous kernel.  The general-purpose version of this kernel (any head size, 32-bit) is
// attention_split.cu; this one exists because the scalar version is bound by instruction issue,
// not by memory.
// FROM_QKV: the kernel takes the qkv product's split partials instead of finished queries, for steps in which
// every request brings one token.  Each CTA sums, norms and rotates the queries of its kv head's group itself
// (every chunk's CTA repeats that: G heads of HD values), and the CTA whose chunk holds the token's own position
// also makes the new key and value row, writes it into its page for later steps and, after a CTA-wide barrier,
// reads it back with the rest of its tile.  This is the q/k kernel's arithmetic (attention.cu: sum in split
// order, round to bfloat16, RMS norm over the head, rotation of pairs (i, i + n_rot/2)) without its launch.
struct QkvSource {
    const float* part;          // [parts][tokens][(nh + 2 nkv) * HD]
    int parts;
    size_t part_stride;
    const float* q_w;           // per-head norm weights, or null: no norm on that side
    const float* k_w;
    const float* inv_freq;      // [n_rot / 2], or null: no rotation
    int n_rot;
    float eps;
    __nv_bfloat16* k_out;       // the caches, writable
    __nv_bfloat16* v_out;
};

template <int HD, bool FROM_QKV>
__global__ void __launch_bounds__(THREADS)
attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                       const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ positions,
                       const int* __restrict__ item_of_token, const int* __restrict__ table, int max_blocks,
                       int page_size, int n_pages, int window, float scale, float* __restrict__ part_acc,
                       float* __restrict__ part_ml, int nh, int nkv, int chunk, int n_splits, int fresh, int overlap_prev,
                       int* status, QkvSource src) {
    constexpr int CH = HD / 8, KT = HD / 16, NT_O = HD / 8;
    constexpr int PER = HD / 32, PAIRS = PER / 2;                  // a head's values per lane; rotation pairs per lane
    extern __shared__ __align__(128) uint8_t pf_smem[];
    __shared__ __align__(16) __nv_bfloat16 q_made[FROM_QKV ? 8 * HD : 8];     // the group's queries, made here
    __shared__ float head_row[FROM_QKV ? 4 : 1][FROM_QKV ? HD : 1];         // a warp's head between norm and rotation
    // shared memory: two buffers of 64 keys and 64 values (32 KB at head size 64, so that four
    // CTAs fit beside a resident product CTA; with three buffers, two of them in flight, fewer CTAs
    // fit an SM and every decode step measured slower); after the key loop the same bytes hold the
    // warps' partial results for the fold
    constexpr int TILE_BYTES = KEYS * HD * 2;
    auto k_s = [&](int buf) { return pf_smem + buf * TILE_BYTES; };          // computed, not an indexed array:
    auto v_s = [&](int buf) { return pf_smem + (2 + buf) * TILE_BYTES; };    // that would live in local memory
    float* wm = reinterpret_cast<float*>(pf_smem);                     // [4][8]
    float* wl = wm + 32;                                               // [4][8]
    float* wacc = wl + 32;                                             // [4][8][HD]
    pdl_trigger();

    // the batch description (positions, block table) comes from the host before the step: it is
    // read, and the chunk's table entries are pulled into the L1, before the wait on the previous kernel
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int G = nh / nkv;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int pos = positions[t];
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int begin = max(lo, split * chunk), end = min(pos + 1, (split + 1) * chunk);
    const int h0 = kvh * G;
    const size_t part_base = ((size_t)t * nh + h0) * n_splits + split;         // + g * n_splits
    const int* tab = table + (size_t)item_of_token[t] * max_blocks;
    const size_t kvw = (size_t)nkv * HD;
    const int kb_first = begin / KEYS, kb_last = (end - 1) / KEYS;
    // A thread fetches half a row of the tile (two threads per key): one page lookup, then CH / 2
    // 16-byte pieces each of the key and of the value.  The two threads of a key take alternate
    // pieces, so that one instruction of the pair covers whole 32-byte sectors.  Warp w fetches keys
    // 16 w .. 16 w + 15 of the tile, the very keys it scores: the key loop needs no CTA-wide barrier.
    auto load_kv = [&](int kb, int buf) {
        static_assert(THREADS == 2 * KEYS, "two threads per key of a tile");
        const int r = tid >> 1, c0 = tid & 1;
        const int j = kb * KEYS + r;
        bool valid = j >= begin && j < end;
        size_t rowi = 0;
        if (valid) {
            // pages of a power of two: shifts, not integer division
            const int blk = page_shift >= 0 ? j >> page_shift : j / page_size;
            const int within = page_shift >= 0 ? j & (page_size - 1) : j % page_size;
            const int page = blk < max_blocks ? tab[blk] : -1;
            if (page < 0 || page >= n_pages) {
                if (c0 == 0) report(status, IMPARO_ST_PAGE_RANGE, 7, t, page);
                valid = false;
            } else {
                rowi = (size_t)page * page_size + within;
            }
        }
        const size_t off = rowi * kvw + (size_t)kvh * HD + c0 * 8;
        uint8_t* const kd = k_s(buf);
        uint8_t* const vd = v_s(buf);
#pragma unroll
        for (int c = 0; c < CH / 2; ++c) {
            cp_async16(kd + tile_off<HD>(r, c0 + 2 * c), k_cache + off + c * 16, valid);
            cp_async16(vd + tile_off<HD>(r, c0 + 2 * c), v_cache + off + c * 16, valid);
        }
        cp_commit();
    };
    // Keys and values at positions below pos + 1 - fresh were written by earlier steps, not by a
    // kernel this one may overlap with (fresh = the most tokens one request brings to this step; 0 =
    // not known): the first two tiles are requested before the wait when they lie there entirely.
    const int old_end = fresh > 0 ? pos + 1 - fresh : -1;
    int requested = kb_first - 1;                                       // tiles asked for so far
    if (begin < end) {
        for (int u = 0; u < 2; ++u) {
            const int kb = kb_first + u;
            if (kb <= kb_last && min(end, (kb + 1) * KEYS) <= old_end) { load_kv(kb, u); requested = kb; } else break;
        }
    }
    // FROM_QKV: the rotation's sines and cosines and the norm weights do not depend on the previous kernel either
    float sn[PAIRS > 0 ? PAIRS : 1], cs[PAIRS > 0 ? PAIRS : 1];
    const int half = FROM_QKV ? src.n_rot >> 1 : 0;
    if (FROM_QKV) {
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            const int i = lane + 32 * j;
            sn[j] = 0.f; cs[j] = 1.f;
            if (src.inv_freq && i < half) sincosf((float)pos * src.inv_freq[i], &sn[j], &cs[j]);
        }
    }
    // overlap_prev: the kernel before this one works on other rows (the step's prompt portions) and let this one start
    // only after its own wait: what this kernel reads is complete, and it runs beside that kernel instead of after it
    if (overlap_prev) pdl_no_wait(); else pdl_wait();
    if (begin >= end) {
        if (tid < G) {
            part_ml[(part_base + (size_t)tid * n_splits) * 2] = -INFINITY;
            part_ml[(part_base + (size_t)tid * n_splits) * 2 + 1] = 0.f;
        }
        if (overlap_prev && tid == 0) pdl_wait_at_end();
        return;
    }

    if (FROM_QKV) {
        // Work items: the group's G query heads; in the CTA whose chunk holds the token's position also the new key
        // (item G) and value (item G + 1).  Warp w takes items w, w + 4, ...; a lane holds the values lane + 32 j.
        const bool owner = pos >= begin && pos < end;
        const int total_w = (nh + 2 * nkv) * HD;
        __nv_bfloat16* kdst = nullptr;
        __nv_bfloat16* vdst = nullptr;
        if (owner) {
            const int blk = page_shift >= 0 ? pos >> page_shift : pos / page_size;
            const int within = page_shift >= 0 ? pos & (page_size - 1) : pos % page_size;
            const int page = blk < max_blocks ? tab[blk] : -1;
            if (page < 0 || page >= n_pages) {
                if (tid == 0) report(status, IMPARO_ST_PAGE_RANGE, 2, t, page);
            } else {
                const size_t r = ((size_t)page * page_size + within) * kvw + (size_t)kvh * HD;
                kdst = src.k_out + r;
                vdst = src.v_out + r;
            }
        }
        const int n_work = G + (owner ? 2 : 0);
        for (int it = warp; it < n_work; it += 4) {
            const bool is_q = it < G, is_k = it == G;
            const int col0 = is_q ? (h0 + it) * HD : (is_k ? (nh + kvh) * HD : (nh + nkv + kvh) * HD);
            const float* ps = src.part + (size_t)t * total_w + col0;
            float val[PER];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int d = lane + 32 * j;
                float acc = 0.f;
                for (int s0 = 0; s0 < src.parts; s0 += 8) {
                    float v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = s0 + u < src.parts ? __ldcg(ps + (size_t)(s0 + u) * src.part_stride + d) : 0.f;
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (s0 + u < src.parts) acc += v[u];
                }
                val[j] = __bfloat162float(__float2bfloat16(acc));             // rounded as the stored product would be
                ss += val[j] * val[j];
            }
            if (is_q || is_k) {
                const float* w = is_q ? src.q_w : src.k_w;
                ss = warp_sum(ss);
                const float nscale = w ? 1.0f / sqrtf(ss / (float)HD + src.eps) : 1.0f;
                float* row = head_row[warp];
#pragma unroll
                for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; row[d] = val[j] * nscale * (w ? w[d] : 1.f); }
                __syncwarp();
                if (src.inv_freq) {
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
                if (is_q) {
#pragma unroll
                    for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; q_made[it * HD + d] = __float2bfloat16(row[d]); }
                } else if (kdst) {
#pragma unroll
                    for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; kdst[d] = __float2bfloat16(row[d]); }
                }
                __syncwarp();                                                  // the row buffer serves the warp's next item
            } else if (vdst) {
#pragma unroll
                for (int j = 0; j < PER; ++j) { const int d = lane + 32 * j; vdst[d] = __float2bfloat16(val[j]); }
            }
        }
        __syncthreads();            // the queries are complete; the new key and value row is visible to this CTA's loads
    }

    // the queries go straight to registers in the MMA's A layout: row g of the 16-row tile is head
    // h0 + g (rows from G up are padding)
    uint32_t qf[KT][4];
    {
        const __nv_bfloat16* qrow = FROM_QKV ? q_made + (g < G ? g : 0) * HD + 2 * tg
                                             : q + ((size_t)t * nh + h0 + (g < G ? g : 0)) * HD + 2 * tg;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            qf[kt][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + kt * 16) : 0u;
            qf[kt][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + kt * 16 + 8) : 0u;
            qf[kt][1] = qf[kt][3] = 0u;
        }
    }
    if (requested < kb_first) {
        load_kv(kb_first, 0);
        requested = kb_first;
    }
    if (tid == 0) timeline_mark(0);
    float o[NT_O][2];                                                   // rows 0..7 only (G <= 8)
#pragma unroll
    for (int n = 0; n < NT_O; ++n) { o[n][0] = o[n][1] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;
    const float sl2 = scale * 1.4426950408889634f;

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int buf = (kb - kb_first) & 1;
        if (kb < kb_last && requested < kb + 1) {
            load_kv(kb + 1, buf ^ 1);
            requested = kb + 1;
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncwarp();                                          // the warp's own 16 keys have landed
        const int mi = lane >> 3, rin = lane & 7;
        const uint8_t* const kt_s = k_s(buf);
        const uint8_t* const vt_s = v_s(buf);
        // this warp's 16 keys of the tile
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        {
            const int key = warp * 16 + (mi >> 1) * 8 + rin;
#pragma unroll
            for (int kt = 0; kt < KT; ++kt) {
                uint32_t b[4];
                ldmatrix4(b, smem_addr(kt_s + tile_off<HD>(key, kt * 2 + (mi & 1))));
                mma16816(s[0], qf[kt], b[0], b[1]);
                mma16816(s[1], qf[kt], b[2], b[3]);
            }
        }
        const int key0 = kb * KEYS + warp * 16 + 2 * tg;
        const int wk0 = kb * KEYS + warp * 16;
        float mx = -INFINITY;
        if (wk0 >= begin && wk0 + 16 <= end) {                  // all 16 keys are live: no masks
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) { s[n][e] *= sl2; mx = fmaxf(mx, s[n][e]); }
        } else {
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = key0 + n * 8 + e;
                    s[n][e] = (j >= begin && j < end) ? s[n][e] * sl2 : -INFINITY;
                    mx = fmaxf(mx, s[n][e]);
                }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m_run, mx);
        const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - mn);
        const float base = (mn == -INFINITY) ? 0.f : mn;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) { s[n][e] = fast_exp2(s[n][e] - base); sum += s[n][e]; }
        l_run = l_run * corr + sum;
        m_run = mn;
        if (__any_sync(0xffffffffu, corr != 1.f)) {             // the running max moved in some row
#pragma unroll
            for (int n = 0; n < NT_O; ++n) { o[n][0] *= corr; o[n][1] *= corr; }
        }
        {
            uint32_t a[4];
            a[0] = pack_bf16(s[0][0], s[0][1]);
            a[1] = 0u;                                                  // rows 8..15 are padding
            a[2] = pack_bf16(s[1][0], s[1][1]);
            a[3] = 0u;
            const int key = warp * 16 + (mi & 1) * 8 + rin;
#pragma unroll
            for (int np = 0; np < NT_O / 2; ++np) {
                uint32_t b[4];
                ldmatrix4_trans(b, smem_addr(vt_s + tile_off<HD>(key, np * 2 + (mi >> 1))));
                float c0[4] = {o[2 * np][0], o[2 * np][1], 0.f, 0.f};
                float c1[4] = {o[2 * np + 1][0], o[2 * np + 1][1], 0.f, 0.f};
                mma16816(c0, a, b[0], b[1]);
                mma16816(c1, a, b[2], b[3]);
                o[2 * np][0] = c0[0]; o[2 * np][1] = c0[1];
                o[2 * np + 1][0] = c1[0]; o[2 * np + 1][1] = c1[1];
            }
        }
        __syncwarp();                                          // the warp refills this buffer two steps on
    }
    __syncthreads();                                           // the tiles' bytes become the fold's scratch
    if (tid == 0) timeline_mark(1);                                     // the key loop is done
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    // ---- fold the four warps (row g = head h0 + g), in warp order ----
    if (tg == 0) { wm[warp * 8 + g] = m_run; wl[warp * 8 + g] = l_run; }
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
        wacc[((size_t)warp * 8 + g) * HD + n * 8 + 2 * tg] = o[n][0];
        wacc[((size_t)warp * 8 + g) * HD + n * 8 + 2 * tg + 1] = o[n][1];
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += THREADS) {
        const int gg = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, wm[w * 8 + gg]);
        float acc = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = wm[w * 8 + gg];
                const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
                acc += wacc[((size_t)w * 8 + gg) * HD + d] * f;
                L += wl[w * 8 + gg] * f;
            }
        }
        const size_t pb = part_base + (size_t)gg * n_splits;
        part_acc[pb * HD + d] = acc;
        // the combine kernel works in natural-log units
        if (d == 0) { part_ml[pb * 2] = M == -INFINITY ? -INFINITY : M * 0.6931471805599453f; part_ml[pb * 2 + 1] = L; }
    }
    if (overlap_prev && tid == 0) pdl_wait_at_end();          // this kernel completes after the one it ran beside
}

}  // namespace pf
}  // namespace imparo

using namespace imparo;

// bfloat16, head size 64 or 128, at most 8 query heads per kv head; else -8 (the caller uses
// another kernel).  n_tok is the batch's token count, n_items its requests.
extern "C" int imparo_attention_prefill(const void* q, const void* k_cache, const void* v_cache,
                                        const int* item_row_start, const int* item_start_pos, int n_items,
                                        const int* table, int max_blocks, int page_size, int n_pages,
                                        int window, float scale, void* out, int n_tok, int nh, int nkv, int hd,
                                        int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0) return -5;
    const int G = nh / nkv;
    if (G > 8 || (hd != 64 && hd != 128)) return -8;
    const int TQ = pf::ROWS / G;
    const long long tiles = (n_tok + TQ - 1) / TQ + n_items;          // an upper bound: every request may end a tile early
    if (tiles > 0x7fffffffLL || nkv > 65535) return -2;
    dim3 grid((unsigned)tiles, nkv);
    cudaError_t e;
    const size_t smem = (size_t)(pf::ROWS + 4 * pf::KEYS) * hd * 2;
    static bool configured = false;
    if (!configured) {
        e = cudaFuncSetAttribute(pf::attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (pf::ROWS + 4 * pf::KEYS) * 128 * 2);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (hd == 64)
        e = launch(pf::attn_prefill_kernel<64>, grid, dim3(pf::THREADS), smem, stream, (const __nv_bfloat16*)q,
                   (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, item_row_start, item_start_pos, n_items, table,
                   max_blocks, page_size, n_pages, window, scale, (__nv_bfloat16*)out, nh, nkv, status);
    else
        e = launch(pf::attn_prefill_kernel<128>, grid, dim3(pf::THREADS), smem, stream, (const __nv_bfloat16*)q,
                   (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, item_row_start, item_start_pos, n_items, table,
                   max_blocks, page_size, n_pages, window, scale, (__nv_bfloat16*)out, nh, nkv, status);
    return e == cudaSuccess ? 0 : (int)e;
}


// Implemented in attention_split.cu: the ordered combine of split partials.
extern "C" int imparo_attention_split_combine(const float* part_acc, const float* part_ml, void* out, int dtype,
                                              int n_rows, int hd, int n_splits, cudaStream_t stream);

// Single query tokens on tensor cores: bfloat16, head size 64 or 128, at most 8 query heads per
// kv head; else -8.  Scratch as for imparo_paged_attention_split.  out == nullptr: the partials are
// left in scratch for a consumer that combines them itself (imparo_gemm_tc_combine).
static int decode_mma_launch(const void* q, const pf::QkvSource* qkv_src, const void* k_cache, const void* v_cache,
                             const int* positions, const int* item_of_token,
                             const int* table, int max_blocks, int page_size, int n_pages,
                             int window, float scale, void* out, float* part_acc, float* part_ml,
                             int n_tok, int nh, int nkv, int hd, int chunk, int n_splits, int fresh, int overlap_prev,
                             int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0) return -5;
    if (nh / nkv > 8 || (hd != 64 && hd != 128)) return -8;
    // at most 2048 splits (the ordered combine keeps one pair per split in shared memory), and the
    // chunks must cover every position a table of this width can hold; refused before any launch
    if (n_tok > 65535 || nkv > 65535 || chunk < 64 || n_splits < 1 || n_splits > 2048) return -2;
    if ((long long)chunk * n_splits < (long long)max_blocks * page_size) return -2;
    dim3 grid(n_splits, nkv, n_tok);
    const size_t smem = (size_t)4 * pf::KEYS * hd * 2;          // the fold's 256 + 128 * hd bytes fit inside
    static bool configured = false;
    cudaError_t e;
    if (!configured) {
        e = cudaFuncSetAttribute(pf::attn_decode_mma_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 4 * pf::KEYS * 128 * 2);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(pf::attn_decode_mma_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     4 * pf::KEYS * 128 * 2);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const bool from_qkv = qkv_src != nullptr;
    const pf::QkvSource none{};
    const pf::QkvSource& src = from_qkv ? *qkv_src : none;
#define IMPARO_DECODE(HD_, F_) launch(pf::attn_decode_mma_kernel<HD_, F_>, grid, dim3(pf::THREADS), smem, stream, \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions, item_of_token, table, \
        max_blocks, page_size, n_pages, window, scale, part_acc, part_ml, nh, nkv, chunk, n_splits, fresh, overlap_prev, status, src)
    if (hd == 64) e = from_qkv ? IMPARO_DECODE(64, true) : IMPARO_DECODE(64, false);
    else e = from_qkv ? IMPARO_DECODE(128, true) : IMPARO_DECODE(128, false);
#undef IMPARO_DECODE
    if (e != cudaSuccess) return (int)e;
    if (out == nullptr) return 0;
    return imparo_attention_split_combine(part_acc, part_ml, out, IMPARO_DT_BF16, n_tok * nh, hd, n_splits, stream);
}

extern "C" int imparo_attention_decode_mma(const void* q, const void* k_cache, const void* v_cache,
                                           const int* positions, const int* item_of_token,
                                           const int* table, int max_blocks, int page_size, int n_pages,
                                           int window, float scale, void* out, float* part_acc, float* part_ml,
                                           int n_tok, int nh, int nkv, int hd, int chunk, int n_splits, int fresh,
                                           int overlap_prev, int* status, cudaStream_t stream) {
    return decode_mma_launch(q, nullptr, k_cache, v_cache, positions, item_of_token, table, max_blocks, page_size, n_pages, window,
                             scale, out, part_acc, part_ml, n_tok, nh, nkv, hd, chunk, n_splits, fresh, overlap_prev ? 1 : 0,
                             status, stream);
}

// The same for a step in which every request brings ONE token, straight from the qkv product's split partials
// (part [parts][n_tok][(nh + 2 nkv) * hd], split s at part + s * part_stride): the queries are made inside the kernel
// and the new key and value rows are written into their pages by it.  q_w / k_w null: no per-head norm on that side;
// inv_freq null: no rotation.  n_rot even, at most hd.
extern "C" int imparo_attention_decode_mma_qkv(const float* part, int parts, long long part_stride, const float* q_w,
                                               const float* k_w, const float* inv_freq, int n_rot, float eps,
                                               void* k_cache, void* v_cache, const int* positions, const int* item_of_token,
                                               const int* table, int max_blocks, int page_size, int n_pages, int window,
                                               float scale, void* out, float* part_acc, float* part_ml, int n_tok, int nh,
                                               int nkv, int hd, int chunk, int n_splits, int* status, cudaStream_t stream) {
    if (part == nullptr || parts < 1) return -24;
    if (n_rot < 0 || (n_rot & 1) || n_rot > hd) return -4;
    pf::QkvSource src{part, parts, (size_t)part_stride, q_w, k_w, inv_freq, inv_freq ? n_rot : 0, eps,
                      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache};
    // fresh = 1: a request's only new row is the one this kernel writes; older rows are safe to request early
    return decode_mma_launch(nullptr, &src, k_cache, v_cache, positions, item_of_token, table, max_blocks, page_size, n_pages,
                             window, scale, out, part_acc, part_ml, n_tok, nh, nkv, hd, chunk, n_splits, 1, 0, status, stream);
}
