// Attention for prompt portions over the paged cache on the 5th-generation tensor cores
// (bfloat16, head size 64 or 128, pages of 16, 32, 64 or 128 positions).
//
// A CTA owns up to 128 query rows: (128 / G) consecutive tokens of ONE request times the G query
// heads that share a kv head (the tile shape of the reference's prefill kernel, "query tokens x GQA
// heads x 1 KV head", imparo-cuda/native/sm80/attention_prefill_mma_d64_f16.cuh:29, at eight times
// its rows).  It walks the keys 128 at a time in position order:
//
//   warp 0      TMA: the step's keys and values, page by page (one tile load per page and 64-dim
//               block, 128-byte swizzle), into a ring of two stages
//   warp 1      tcgen05.mma: S = Q K^T into tensor memory (M = 128 rows, N = 128 keys), and, once
//               the softmax warps have written P, O_step = P V (M = 128, N = head size), the values
//               read as they lie in the cache (MN-major operand)
//   warps 2-9   two threads per row (half of the step's keys and half of the head's dims each): read S
//               from tensor memory, mask by position and window, running max and sum in 32-bit,
//               P = exp2(s - max) as bfloat16 into shared memory in the MMA's swizzled layout; read
//               O_step and fold it into the row's 32-bit output registers
//
// Formulas: scores q.k * scale for lo <= key <= position, lo = 0 or position + 1 - window, no mask
// tensor, softmax with the max subtracted (imparo-model/src/cpu_support.rs:402-445).  Which tokens
// form a tile is derived on the device from the batch's row starts, so a tile never holds rows of
// two requests; a row's result does not depend on its neighbours in the tile.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records IMPARO_ST_WAIT_LIMIT in
// the status word, stops waiting, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace imparo {
namespace fa {

using namespace tc;

constexpr int ROWS = 128;          // query rows per CTA: the MMAs' M
constexpr int KEYS = 128;          // keys per step: N of the score product, K of P V
constexpr int THREADS = 320;       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-9: softmax
constexpr int STAGES = 2;
constexpr uint32_t REGION = 128 * 128;      // a [128 rows][128 bytes] block of a tile: 16 KB
constexpr uint32_t ALIGN_SLACK = 768;       // spare bytes for aligning the tiles to 1024: two CTAs must fit an SM at head size 64

// The values as B operand: [key][dim] with the dims contiguous (MN-major), 128-byte swizzle:
// groups of 8 keys are 1024 bytes apart (SBO), 64-dim blocks lbo bytes apart.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, bfloat16 operands, float32 accumulator; b_mn: the B operand is MN-major
__device__ __forceinline__ uint32_t instr_desc_ab(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// 2^x for x <= 0 (scores minus their max): the hardware approximation, one instruction
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// one 32-bit value per lane into a tensor-memory column, and a pair of neighbouring columns back
__device__ __forceinline__ void tmem_st1(uint32_t taddr, float v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(__float_as_uint(v)) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld2(uint32_t taddr, float& x, float& y) {
    uint32_t r0, r1;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    asm volatile("" : "+r"(r0), "+r"(r1) :: "memory");
    x = __uint_as_float(r0);
    y = __uint_as_float(r1);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Args {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* item_row_start;
    const int* item_start_pos;
    const int* table;
    int* status;
    int n_items, max_blocks, page_size, n_pages, window, nh, nkv;
    float scale;
    int late_trigger;        // the next kernel runs beside this one and must find all before this one complete (common.cuh)
};

template <int HD>
__global__ void __launch_bounds__(THREADS, HD == 64 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a) {
    constexpr int NB = HD / 64;                              // 64-dim blocks of a head
    constexpr uint32_t Q_BYTES = NB * REGION, P_BYTES = 2 * REGION, K_BYTES = NB * REGION, V_BYTES = NB * REGION;
    constexpr uint32_t STAGE_BYTES = K_BYTES + V_BYTES;
    constexpr uint32_t TMEM_COLS = HD == 64 ? 256 : 512;     // scores: columns 0..127, P V: 128..128+HD-1, then four spare
    constexpr uint32_t XCOL = 128 + HD;                      // columns the two threads of a row exchange through
    extern __shared__ __align__(1024) uint8_t fa_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)fa_smem_raw + 1023) & ~(uintptr_t)1023);
    if ((uint32_t)(smem - fa_smem_raw) > ALIGN_SLACK) {      // the launch's shared memory does not cover the aligned tiles
        if (threadIdx.x == 0) report(a.status, IMPARO_ST_WAIT_LIMIT, 29, (int)(smem - fa_smem_raw), 0);
        return;
    }
    uint8_t* q_s = smem;
    uint8_t* p_s = q_s + Q_BYTES;
    uint8_t* kv_s = p_s + P_BYTES;                           // [stage][K | V]
    uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + STAGES * STAGE_BYTES);
    uint64_t* kv_full = bars;                                // [STAGES]
    uint64_t* kv_empty = bars + STAGES;                      // [STAGES]
    uint64_t* q_ready = bars + 2 * STAGES;
    uint64_t* s_ready = q_ready + 1;
    uint64_t* p_ready = q_ready + 2;
    uint64_t* pv_ready = q_ready + 3;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 4);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);     // a softmax thread's wait ran out

    if (a.late_trigger) { timeline_begin(); pdl_wait(); pdl_trigger_late(); } else pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = a.nh / a.nkv;
    const int TQ = ROWS / G;                                 // tokens per tile
    // The kv head is the fast grid index and the tiles run backwards along the slow one: CTAs are
    // handed out in that order, so the tiles with the most keys under a causal mask start first
    // and the short ones fill the SMs' last gaps.
    const int kvh = blockIdx.x;
    // which request and which of its tokens: tiles are numbered request by request
    int item = 0, tile = (int)gridDim.y - 1 - (int)blockIdx.y, n_item = 0, row0 = 0;
    for (; item < a.n_items; ++item) {
        row0 = a.item_row_start[item];
        n_item = a.item_row_start[item + 1] - row0;
        const int tiles = (n_item + TQ - 1) / TQ;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (item >= a.n_items) {                                 // the grid is an upper bound (uniform per CTA)
        if (threadIdx.x == 0) pdl_wait();                    // (keeps the launch's timeline record whole)
        return;
    }
    const int tok0 = tile * TQ;
    const int n_tok = min(TQ, n_item - tok0);
    const int n_rows = n_tok * G;
    const int pos0 = a.item_start_pos[item] + tok0;
    const int pos_last = pos0 + n_tok - 1;
    const int* tab = a.table + (size_t)item * a.max_blocks;
    const int lo_min = (a.window > 0 && pos0 + 1 > a.window) ? pos0 + 1 - a.window : 0;
    const int kb_first = lo_min / KEYS, kb_last = pos_last / KEYS;
    const int n_steps = kb_last - kb_first + 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(q_ready, 256);
        mbar_init(s_ready, 1);
        mbar_init(p_ready, 256);
        mbar_init(pv_ready, 1);
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- keys and values, page by page: lane 0 waits for the stage and sets the byte count, lane p then looks up
        // page p of the step in the block table and issues that page's copies (one thread walking the pages pays a
        // dependent table read per page) ----
        pdl_wait();                                          // this step's keys were written by the kernel before
        const int pages_per_step = KEYS / a.page_size;
        const int first_blk = lo_min / a.page_size, last_blk = pos_last / a.page_size;
        for (int i = 0; i < n_steps; ++i) {
            const int s = i % STAGES;
            int ok = 1;
            if (lane == 0) {
                if (i >= STAGES && !mbar_wait(&kv_empty[s], ((i / STAGES) - 1) & 1)) {
                    report(a.status, IMPARO_ST_WAIT_LIMIT, 20, i, s);
                    ok = 0;
                } else {
                    mbar_expect_tx(&kv_full[s], STAGE_BYTES);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);            // (also orders the byte count before the copies)
            if (!ok) break;
            uint8_t* kdst = kv_s + s * STAGE_BYTES;
            uint8_t* vdst = kdst + K_BYTES;
            const int blk0 = (kb_first + i) * pages_per_step;
            for (int pg = lane; pg < pages_per_step; pg += 32) {
                // blocks before every row's window or past the request's last position hold nothing
                // this tile may use (a window's old pages may be gone): a mapped page stands in
                // for them (their keys are masked, their values finite)
                const int blk = min(max(blk0 + pg, first_blk), last_blk);
                int page = blk < a.max_blocks ? tab[blk] : -1;
                if (page < 0 || page >= a.n_pages) {
                    report(a.status, IMPARO_ST_PAGE_RANGE, 21, item, page);
                    page = 0;
                }
                const int y = page * a.page_size;
                const uint32_t off = (uint32_t)pg * a.page_size * 128;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    tma_load_2d(kdst + nb * REGION + off, &map_k, &kv_full[s], kvh * HD + nb * 64, y);
                    tma_load_2d(vdst + nb * REGION + off, &map_v, &kv_full[s], kvh * HD + nb * 64, y);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- the two products of every step ----
            const uint32_t idesc_s = instr_desc_ab(ROWS, KEYS, false);
            const uint32_t idesc_o = instr_desc_ab(ROWS, HD, true);
            const uint32_t t_s = tmem_base, t_o = tmem_base + 128;
            bool ok = mbar_wait(q_ready, 0);
            if (!ok) report(a.status, IMPARO_ST_WAIT_LIMIT, 22, 0, 0);
            auto issue_pv = [&](int i) {                      // O_step = P_i V_i
                const uint32_t vb = smem_u32(kv_s + (i % STAGES) * STAGE_BYTES + K_BYTES), pb = smem_u32(p_s);
#pragma unroll
                for (int kk = 0; kk < KEYS / UMMA_K; ++kk)
                    umma(t_o, smem_desc(pb + (kk >> 2) * REGION + (kk & 3) * 32), smem_desc_mn(vb + kk * (UMMA_K * 128), REGION),
                         idesc_o, kk > 0 ? 1u : 0u);
                umma_commit(&kv_empty[i % STAGES]);          // keys (scored earlier) and values of the stage are read
                umma_commit(pv_ready);
            };
            for (int i = 0; i < n_steps && ok; ++i) {
                // P of the step before is written and its scores are read: the score tile is free again
                if (i > 0 && !mbar_wait(p_ready, (i - 1) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 23, i, 0); ok = false; break; }
                const int s = i % STAGES;
                if (!mbar_wait(&kv_full[s], (i / STAGES) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 24, i, s); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t qb = smem_u32(q_s), kb = smem_u32(kv_s + s * STAGE_BYTES);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma(t_s, smem_desc(qb + nb * REGION + k * 32), smem_desc(kb + nb * REGION + k * 32), idesc_s,
                             (nb > 0 || k > 0) ? 1u : 0u);
                umma_commit(s_ready);                        // the softmax warps want this first ...
                if (i > 0) issue_pv(i - 1);                  // ... the step before's P V only when they fold it
            }
            if (ok) {
                if (mbar_wait(p_ready, (n_steps - 1) & 1)) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_pv(n_steps - 1);
                } else {
                    report(a.status, IMPARO_ST_WAIT_LIMIT, 25, n_steps, 0);
                }
            }
        }
    } else {
        // ---- softmax: two threads per row (= tensor-memory lane), one for each half of the step's keys
        // and of the head's dims.  Warps 2-5 take keys 0-63, warps 6-9 keys 64-127; the two threads of a
        // row agree on the row's max through two spare tensor-memory columns.
        const int half = (warp - 2) >> 2;
        const int r = (warp & 3) * 32 + lane;
        const bool valid = r < n_rows;
        const int tok = r / G, head = kvh * G + r % G;
        const int pos_r = pos0 + tok;
        const int lo_r = (a.window > 0 && pos_r + 1 > a.window) ? pos_r + 1 - a.window : 0;
        const int lo_last = (a.window > 0 && pos_last + 1 > a.window) ? pos_last + 1 - a.window : 0;
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t t_s = t_lane + half * 64, t_o = t_lane + 128 + half * (HD / 2), t_x = t_lane + XCOL;
        const size_t row_off = ((size_t)(row0 + tok0 + (valid ? tok : 0)) * a.nh + head) * HD;
        constexpr int DH = HD / 2;                           // dims of the output this thread keeps
        pdl_wait();
        // this thread's half of the row's queries -> shared memory, 16-byte chunks swizzled as the MMA reads them
        {
            const uint4* src = reinterpret_cast<const uint4*>(a.q + row_off);
#pragma unroll
            for (int cc = 0; cc < DH / 8; ++cc) {
                const int c = half * (DH / 8) + cc;
                const uint4 v = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(q_s + (c >> 3) * REGION + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(q_ready)) : "memory");
        }
        float o[DH];
#pragma unroll
        for (int d = 0; d < DH; ++d) o[d] = 0.f;
        float m_run = -INFINITY, l_run = 0.f, corr_prev = 0.f;
        const float sl2 = a.scale * 1.4426950408889634f;     // scores in units of log2(e)
        bool ok = true;
        auto fold_pv = [&](float corr) {                     // o = o * corr + O_step (this thread's dims)
#pragma unroll
            for (int c = 0; c < DH; c += 32) {
                float v[2][16];
                tmem_ld_chunks<2>(t_o + c, v);
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int e = 0; e < 16; ++e) o[c + u * 16 + e] = o[c + u * 16 + e] * corr + v[u][e];
            }
        };
        for (int i = 0; i < n_steps; ++i) {
            const int key0 = (kb_first + i) * KEYS + half * 64;          // this thread's first key of the step
            // A wait that runs out is recorded; every softmax thread still goes through the same named
            // barriers and all leave together after the next one.
            if (!mbar_wait(s_ready, i & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 26, i, r); *gave_up = 1; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // which of its 64 keys this row sees: [j_lo, j_hi] relative to key0 (empty for padding rows).
            // A step that every row of the tile sees whole (all but the steps at the diagonal and at a
            // window's edge) skips the per-key tests.
            const int j_hi = valid ? min(63, pos_r - key0) : -1;
            const int j_lo = max(0, lo_r - key0);
            const bool whole = (kb_first + i) * KEYS + KEYS - 1 <= pos0 && (kb_first + i) * KEYS >= lo_last;
            // pass 1: the max over this thread's keys (four running maxima: no long dependent chain)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v[2][16];
                tmem_ld_chunks<2>(t_s + h * 32, v);
                if (whole) {
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int e = 0; e < 16; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], v[u][e]);
                } else {
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int j = h * 32 + u * 16 + e;
                            if (j >= j_lo && j <= j_hi) mx4[e & 3] = fmaxf(mx4[e & 3], v[u][e]);
                        }
                }
            }
            // the row's max: both threads of the row leave theirs in tensor memory and read the pair
            tmem_st1(t_x + half, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 256;" ::: "memory");
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (*gave_up) { ok = false; break; }
            float mx_a, mx_b;
            tmem_ld2(t_x, mx_a, mx_b);
            const float mx = fmaxf(mx_a, mx_b) * sl2;        // sl2 > 0: the max commutes with the scaling
            const float m_new = fmaxf(m_run, mx);
            const float corr = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_new);
            const float base = (m_new == -INFINITY) ? 0.f : m_new;
            // the previous step's P V is complete by now or soon: fold it in before P is overwritten
            if (i > 0) {
                if (!mbar_wait(pv_ready, (i - 1) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 27, i, r); *gave_up = 1; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                fold_pv(corr_prev);
            }
            // pass 2: P = exp2(s - max), bfloat16, into shared memory; this thread's share of the row's sum
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            const float nbase = -base;
            uint8_t* prow = p_s + half * REGION + r * 128;   // keys 0-63 and 64-127 are the two blocks of P
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v[2][16];
                tmem_ld_chunks<2>(t_s + h * 32, v);
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    uint32_t w[8];
                    if (whole) {
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            const float p0 = ex2(fmaf(v[u][e], sl2, nbase)), p1 = ex2(fmaf(v[u][e + 1], sl2, nbase));
                            sum4[(e >> 1) & 3] += p0 + p1;
                            w[e >> 1] = pack2(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            const int j = h * 32 + u * 16 + e;
                            const float p0 = (j >= j_lo && j <= j_hi) ? ex2(fmaf(v[u][e], sl2, nbase)) : 0.f;
                            const float p1 = (j + 1 >= j_lo && j + 1 <= j_hi) ? ex2(fmaf(v[u][e + 1], sl2, nbase)) : 0.f;
                            sum4[(e >> 1) & 3] += p0 + p1;
                            w[e >> 1] = pack2(p0, p1);
                        }
                    }
                    // keys h*32 + u*16 .. +15 of this block: chunks 4h + 2u and 4h + 2u + 1 of the row's 128 bytes
                    const int c0 = 4 * h + 2 * u;
                    *reinterpret_cast<uint4*>(prow + ((c0 ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(prow + (((c0 + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
            l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            m_run = m_new;
            corr_prev = corr;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(p_ready)) : "memory");
        }
        if (ok) {                                            // uniform over the softmax threads (set after a barrier)
            if (!mbar_wait(pv_ready, (n_steps - 1) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 28, n_steps, r); *gave_up = 1; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            fold_pv(corr_prev);
            // the row's sum: the two threads' shares, in the order (keys 0-63, keys 64-127)
            tmem_st1(t_x + 2 + half, l_run);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 256;" ::: "memory");
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float l_a, l_b;
            tmem_ld2(t_x + 2, l_a, l_b);
            const float l = l_a + l_b;
            if (valid && !*gave_up) {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                uint4* dst = reinterpret_cast<uint4*>(a.out + row_off + half * DH);
#pragma unroll
                for (int c = 0; c < DH / 8; ++c)
                    dst[c] = make_uint4(pack2(o[c * 8] * inv, o[c * 8 + 1] * inv), pack2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv),
                                        pack2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv), pack2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int HD>
static int launch_tc(const CUtensorMap& mk, const CUtensorMap& mv, const Args& a, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = ALIGN_SLACK + (size_t)(HD / 64) * REGION + 2 * REGION + (size_t)STAGES * 2 * (HD / 64) * REGION + 128;
    auto kern = attn_prefill_tc_kernel<HD>;
    static bool configured = false;
    cudaError_t e;
    if (!configured) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    e = launch(kern, grid, dim3(THREADS), smem, stream, mk, mv, a);
    return e == cudaSuccess ? 0 : (int)e;
}


// ---- two query tiles per CTA in turn (head size 64) ------------------------------------------------
// The kernel above does the two products and the softmax of a step one after the other; the tensor cores wait while
// the softmax runs.  Here a CTA owns TWO query tiles of 128 rows (consecutive tokens of one request, the same kv
// head) and ONE stream of keys and values that both use:
//
//   warp 0      TMA: keys and values page by page into rings of three buffers each (lane p fetches page p of a step;
//               keys and values have barriers of their own, since a step's keys are read long before its values)
//   warp 1, 18  tcgen05.mma, one issuing thread per tile: S_x = Q_x K^T into the tile's 128 score columns of tensor
//               memory, issued for the NEXT step as soon as the softmax has read the current scores, and
//               O_x += P_x V accumulated IN tensor memory, issued when the step's probabilities are written
//   warps 2-9   softmax of tile A, warps 10-17 of tile B: two threads per row, one for each half of the step's keys
//               and of the head's dims.  A thread's 64 scores of the step go to registers in one sweep (the score
//               columns are free for the next step's product at once), the two threads of a row agree on the row's
//               max through shared memory, P = exp2(s - max) goes to shared memory as bfloat16 in the MMA's layout.
// The two tiles take turns at the exponential pass (a barrier each way): the exp2 units are what both softmaxes need
// at full rate, and with the passes apart one tile's products, loads and max run under the other tile's pass.
// What the device's clock showed while this was shaped (stamps per phase in one CTA, a temporary build): one thread
// issuing for both tiles was busy the whole step (an instruction of this size keeps its thread 70-120 cycles, 24 per
// step of both tiles), one thread walking a step's pages paid eight dependent table reads in a row, and two exp passes
// at once took 2,500 cycles each where one alone takes 1,400.
// The output stays in tensor memory across steps.  When a row's max grows, what has been accumulated must be scaled
// down; that costs a round trip of the row's output through registers, so it is done only when the max has grown by
// more than 8 (in log2 units: a factor of 256) in some row of the warp; otherwise the old max stays in use, the
// exponentials are at most 256, and the final division by the row's sum (taken with the same max) gives the same
// result.  Formulas and masks as above.
constexpr int PP_THREADS = 608;     // warp 0: TMA, warp 1: tile A's products + tensor memory, warps 2-9: softmax of tile A, 10-17: of tile B, 18: tile B's products
constexpr int PP_MMA_B_WARP = 18;
constexpr int PP_STAGES = 3;
constexpr float PP_GROW = 8.0f;

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void keep32(uint32_t (&r)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(r[i]) :: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(PP_THREADS, 1)
attn_prefill_pp_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a) {

    constexpr int HD = 64;
    constexpr uint32_t Q_BYTES = REGION, P_BYTES = 2 * REGION, STAGE_BYTES = 2 * REGION;      // per tile; per stage K | V
    constexpr uint32_t TMEM_COLS = 512;                      // scores of A, of B: 0..127, 128..255; outputs: 256.., 320..
    extern __shared__ __align__(1024) uint8_t fa_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)fa_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                                     // [2][Q_BYTES]
    uint8_t* p_s = q_s + 2 * Q_BYTES;                        // [2][P_BYTES]
    uint8_t* kv_s = p_s + 2 * P_BYTES;                       // [stage][K | V]
    uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + PP_STAGES * STAGE_BYTES);
    // Keys and values of a step have barriers of their own: a step's keys are read last by the score products, which
    // are issued a whole softmax before the step's P V products, so their buffer is free that much earlier
    uint64_t* k_full = bars;                                 // [PP_STAGES]
    uint64_t* k_empty = k_full + PP_STAGES;                  // [PP_STAGES]
    uint64_t* q_ready = k_empty + PP_STAGES;
    uint64_t* s_ready = q_ready + 1;                         // [2]  the tile's scores of a step are complete
    uint64_t* s_free = s_ready + 2;                          // [2]  ... and have been read into registers
    uint64_t* p_ready = s_free + 2;                          // [2]  P of the step is in shared memory, the output scaled
    uint64_t* o_done = p_ready + 2;                          // [2]  P V of the step is accumulated
    uint64_t* v_full = o_done + 2;                           // [PP_STAGES]
    uint64_t* v_empty = v_full + PP_STAGES;                  // [PP_STAGES]
    // The two tiles take turns at the exponential: the SM's exp2 units are the one resource both softmaxes need at
    // full rate, and when both tiles' passes coincide each takes twice as long while the units idle for the rest of
    // the step.  turn[x] completes when the OTHER tile has finished a pass and tile x may start its next one.
    uint64_t* turn = v_empty + PP_STAGES;                    // [2]
    uint64_t* p_half = turn + 2;                             // [2]  every thread's first 32 probabilities of the step are written
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_half + 2);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(bars) + 64;        // [tile][buffer][half][row]: what the two threads of a row exchange
    static_assert((4 * PP_STAGES + 13) * 8 + 8 <= 256, "barriers overlap the exchange buffer");

    if (a.late_trigger) { timeline_begin(); pdl_wait(); pdl_trigger_late(); } else pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = a.nh / a.nkv;
    const int TQ = ROWS / G;                                 // tokens per tile; a CTA takes two tiles
    const int kvh = blockIdx.x;
    int item = 0, pair = (int)gridDim.y - 1 - (int)blockIdx.y, n_item = 0, row0 = 0;
    for (; item < a.n_items; ++item) {
        row0 = a.item_row_start[item];
        n_item = a.item_row_start[item + 1] - row0;
        const int pairs = (n_item + 2 * TQ - 1) / (2 * TQ);
        if (pair < pairs) break;
        pair -= pairs;
    }
    if (item >= a.n_items) {                                 // the grid is an upper bound (uniform per CTA)
        if (threadIdx.x == 0) pdl_wait();
        return;
    }
    // tile x: tokens tok0[x] .. tok0[x] + n_tok[x] - 1 of the request
    const int tokA = pair * 2 * TQ;
    const int n_tokA = min(TQ, n_item - tokA), n_tokB = max(0, min(TQ, n_item - tokA - TQ));
    const int start = a.item_start_pos[item];
    const int posA0 = start + tokA, pos_lastA = posA0 + n_tokA - 1;
    const int posB0 = posA0 + TQ, pos_lastB = posB0 + n_tokB - 1;
    const int* tab = a.table + (size_t)item * a.max_blocks;
    const int lo_min = (a.window > 0 && posA0 + 1 > a.window) ? posA0 + 1 - a.window : 0;
    const int kb_first = lo_min / KEYS;
    const int nA = pos_lastA / KEYS - kb_first + 1;
    const int nB = n_tokB > 0 ? pos_lastB / KEYS - kb_first + 1 : 0;
    const int n_steps = max(nA, nB);
    const int pos_last = n_tokB > 0 ? pos_lastB : pos_lastA;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PP_STAGES; ++s) {
            // a buffer is free when every tile that exists has read it
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], nB > 0 ? 2 : 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], nB > 0 ? 2 : 1);
        }
        mbar_init(q_ready, 512);
        mbar_init(&turn[0], 256); mbar_init(&turn[1], 256);
        mbar_init(&p_half[0], 256); mbar_init(&p_half[1], 256);
        for (int x = 0; x < 2; ++x) { mbar_init(&s_ready[x], 1); mbar_init(&s_free[x], 256); mbar_init(&p_ready[x], 256); mbar_init(&o_done[x], 1); }
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // The whole warp fetches: lane 0 looks at the barriers and sets the byte count, then lane p looks up page p of
        // the step in the block table and issues that page's copy.  (One thread walking the pages paid a dependent
        // table read per page, eight in a row for pages of 16: about as long as a whole step of the softmax.)
        pdl_wait();                                          // this step's keys were written by the kernel before
        const int pages_per_step = KEYS / a.page_size;
        const int first_blk = lo_min / a.page_size, last_blk = pos_last / a.page_size;
        auto load = [&](int i, bool values) {                // warp-uniform call
            const int s = i % PP_STAGES;
            uint8_t* dst = kv_s + s * STAGE_BYTES + (values ? REGION : 0);
            uint64_t* bar = values ? &v_full[s] : &k_full[s];
            if (lane == 0) mbar_expect_tx(bar, REGION);
            __syncwarp();
            const int blk0 = (kb_first + i) * pages_per_step;
            for (int pg = lane; pg < pages_per_step; pg += 32) {
                const int blk = min(max(blk0 + pg, first_blk), last_blk);       // (see the kernel above)
                int page = blk < a.max_blocks ? tab[blk] : -1;
                if (page < 0 || page >= a.n_pages) {
                    report(a.status, IMPARO_ST_PAGE_RANGE, 41, item, page);
                    page = 0;
                }
                tma_load_2d(dst + (uint32_t)pg * a.page_size * 128, values ? &map_v : &map_k, bar, kvh * HD, page * a.page_size);
            }
        };
        // keys and values are fetched as their buffers come free, whichever first
        int k_next = 0, v_next = 0;
        uint32_t idle = 0;
        while (k_next < n_steps || v_next < n_steps) {
            int what = 0;                                    // bit 0: the next keys' buffer is free, bit 1: the next values', bit 2: stop
            if (lane == 0) {
                if (k_next < n_steps && (k_next < PP_STAGES || mbar_test(&k_empty[k_next % PP_STAGES], ((k_next / PP_STAGES) - 1) & 1))) what |= 1;
                if (v_next < n_steps && (v_next < PP_STAGES || mbar_test(&v_empty[v_next % PP_STAGES], ((v_next / PP_STAGES) - 1) & 1))) what |= 2;
                if (*gave_up) what = 4;
                if (what == 0 && ++idle > WAIT_LIMIT / 16) {
                    report(a.status, IMPARO_ST_WAIT_LIMIT, 40, k_next, v_next);
                    *gave_up = 1;
                    what = 4;
                }
            }
            what = __shfl_sync(0xffffffffu, what, 0);
            if (what & 4) break;
            if (what & 1) load(k_next++, false);
            if (what & 2) load(v_next++, true);
            if (what != 0) idle = 0; else __nanosleep(200);      // (not urgent: a buffer is free a period or more before it is needed)
        }
    } else if (warp == 1 || warp == PP_MMA_B_WARP) {
        // One issuing thread per tile (warp 1: tile A, the last warp: tile B).  A tensor-core instruction of this size
        // (128 x 128 x 16 for the scores, 128 x 64 x 16 for P V) keeps its issuing thread for 70 to 90 cycles, 24 of them
        // per step of both tiles: one thread serving both tiles was busy the whole step and every product came late.
        // A tile's thread issues the tile's NEXT scores as soon as the softmax has read the current ones (s_free), a
        // whole softmax before they are needed, and the tile's P V product when its probabilities are written
        // (p_ready); the waits block (a thread that polls takes issue slots from the softmax warps of its scheduler).
        // A step's keys are free when both tiles' score products are issued, its values when both P V products are:
        // each thread commits to those barriers after its own product (they count the tiles).
        const int x = warp == 1 ? 0 : 1;
        const int n_x = x == 0 ? nA : nB;
        if (lane == 0 && (n_x > 0 || x == 0)) {
            const uint32_t idesc_s = instr_desc_ab(ROWS, KEYS, false);
            const uint32_t idesc_o = instr_desc_ab(ROWS, HD, true);
            bool ok = mbar_wait(q_ready, 0);
            if (!ok) { report(a.status, IMPARO_ST_WAIT_LIMIT, 42, x, 0); *gave_up = 1; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int k_seen = -1, v_seen = -1;                    // steps whose keys / values have landed
            auto wait_or_give_up = [&](uint64_t* bar, uint32_t parity, int code, int j) -> bool {
                if (mbar_wait(bar, parity)) { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); return true; }
                report(a.status, IMPARO_ST_WAIT_LIMIT, code, j, x);
                *gave_up = 1;
                return false;
            };
            auto need_keys = [&](int j) -> bool {
                while (k_seen < j) {
                    const int i = k_seen + 1;
                    if (!wait_or_give_up(&k_full[i % PP_STAGES], (i / PP_STAGES) & 1, 43, i)) return false;
                    k_seen = i;
                }
                return true;
            };
            auto need_values = [&](int j) -> bool {
                while (v_seen < j) {
                    const int i = v_seen + 1;
                    if (!wait_or_give_up(&v_full[i % PP_STAGES], (i / PP_STAGES) & 1, 49, i)) return false;
                    v_seen = i;
                }
                return true;
            };
            // The descriptors of the buffers are made once; an operand at a byte offset inside a buffer is its
            // descriptor plus offset / 16 (the address field is the low 14 bits and never carries: shared memory is
            // smaller than that), with offsets the compiler knows.
            const uint64_t qd = smem_desc(smem_u32(q_s + x * Q_BYTES)), dk0 = smem_desc(smem_u32(kv_s));
            const uint64_t pd = smem_desc(smem_u32(p_s + x * P_BYTES)), dv0 = smem_desc_mn(smem_u32(kv_s + REGION), REGION);
            const uint32_t t_s = tmem_base + x * 128, t_o = tmem_base + 256 + x * HD;
            auto issue_s = [&](int j) {                      // S_x = Q_x K_j^T
                const uint64_t kd = dk0 + (uint64_t)(((j % PP_STAGES) * STAGE_BYTES) >> 4);
                umma(t_s, qd, kd, idesc_s, 0u);
#pragma unroll
                for (int k = 1; k < BK / UMMA_K; ++k) umma(t_s, qd + (uint64_t)((k * 32) >> 4), kd + (uint64_t)((k * 32) >> 4), idesc_s, 1u);
                umma_commit(&s_ready[x]);
                umma_commit(&k_empty[j % PP_STAGES]);        // this tile has read the step's keys when the product has run
            };
            // O_x (+)= P_x V_j in two halves: a softmax thread writes the probabilities of its first 32 keys, then of its
            // second 32 (the two threads of a row own keys 0-63 and 64-127), so keys 0-31 and 64-95 are there first.  Their
            // share of the product is issued then, under the softmax's second half, and the product is done sooner after
            // the step's end.
            auto issue_pv_half = [&](int j, const int h) {
                const uint64_t vd = dv0 + (uint64_t)(((j % PP_STAGES) * STAGE_BYTES) >> 4);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int kk = (u >> 1) * 4 + 2 * h + (u & 1);           // 16 keys each: 0, 1, 4, 5 then 2, 3, 6, 7
                    umma(t_o, pd + (uint64_t)(((kk >> 2) * REGION + (kk & 3) * 32) >> 4), vd + (uint64_t)((kk * (UMMA_K * 128)) >> 4), idesc_o,
                         (kk > 0 || j > 0) ? 1u : 0u);
                }
                if (h == 1) {
                    umma_commit(&o_done[x]);
                    umma_commit(&v_empty[j % PP_STAGES]);
                }
            };
            if (ok && n_x > 0 && need_keys(0)) issue_s(0); else ok = ok && n_x == 0;
            for (int j = 0; j < n_x && ok; ++j) {
                if (j + 1 < n_x) {
                    ok = wait_or_give_up(&s_free[x], j & 1, 45, j) && need_keys(j + 1);
                    if (!ok) break;
                    issue_s(j + 1);
                }
                ok = wait_or_give_up(&p_half[x], j & 1, 51, j) && need_values(j);
                if (!ok) break;
                issue_pv_half(j, 0);
                ok = wait_or_give_up(&p_ready[x], j & 1, 44, j);
                if (!ok) break;
                issue_pv_half(j, 1);
            }
            // Tile B may have one step more than tile A (its positions lie behind A's); A's thread then gives that
            // step's keys and values free on its own behalf, having no product that reads them.
            // (Only once that step's keys and values have landed: their buffers' earlier contents are then surely
            // given free by both tiles, so this thread's two arrivals on a barrier cannot fall into one phase.)
            if (ok && x == 0 && nB > nA && need_keys(nA) && need_values(nA)) {
                umma_commit(&k_empty[nA % PP_STAGES]);
                umma_commit(&v_empty[nA % PP_STAGES]);
            }
        }
    } else {
        // ---- softmax: two threads per row of tile x, one for each half of the step's keys and of the head's dims ----
        const int x = (warp - 2) >> 3;
        const int half = ((warp - 2) >> 2) & 1;
        const int r = (warp & 3) * 32 + lane;
        const int n_x = x == 0 ? nA : nB;
        const int n_rows = (x == 0 ? n_tokA : n_tokB) * G;
        const bool valid = r < n_rows;
        const int tok = r / G, head = kvh * G + r % G;
        const int pos0 = x == 0 ? posA0 : posB0;
        const int pos_r = pos0 + tok;
        const int pos_last_x = x == 0 ? pos_lastA : pos_lastB;
        const int lo_r = (a.window > 0 && pos_r + 1 > a.window) ? pos_r + 1 - a.window : 0;
        const int lo_last = (a.window > 0 && pos_last_x + 1 > a.window) ? pos_last_x + 1 - a.window : 0;
        const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t t_s = t_lane + x * 128 + half * 64, t_o = t_lane + 256 + x * HD + half * (HD / 2);
        const size_t row_off = ((size_t)(row0 + tokA + x * TQ + (valid ? tok : 0)) * a.nh + head) * HD;
        float* my_x = xch + ((x * 2 + 0) * 2 + half) * ROWS + r;              // [tile][buffer][half][row]
        float* other_x = xch + ((x * 2 + 0) * 2 + (half ^ 1)) * ROWS + r;
        pdl_wait();
        {
            // this thread's half of the row's queries -> shared memory, 16-byte chunks swizzled as the MMA reads them
            const uint4* src = reinterpret_cast<const uint4*>(a.q + row_off);
#pragma unroll
            for (int cc = 0; cc < HD / 16; ++cc) {
                const int c = half * (HD / 16) + cc;
                const uint4 v = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(q_s + x * Q_BYTES + r * 128 + ((c ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(q_ready);
        }
        float m_used = -INFINITY, l_run = 0.f;
        const float sl2 = a.scale * 1.4426950408889634f;     // scores in units of log2(e)
        bool ok = true;
        uint8_t* prow = p_s + x * P_BYTES + half * REGION + r * 128;         // keys 0-63 and 64-127 are the two blocks of P
        for (int j = 0; j < n_x; ++j) {
            if (!mbar_wait(&s_ready[x], j & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 46, j, r); *gave_up = 1; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sv[2][32];                              // this thread's 64 scores of the step
            tmem_ld32_nowait(t_s, sv[0]);
            tmem_ld32_nowait(t_s + 32, sv[1]);
            tmem_wait_ld();
            keep32(sv[0]); keep32(sv[1]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&s_free[x]);                         // the score columns may take the next step's product
            const int key0 = (kb_first + j) * KEYS + half * 64;              // this thread's first key of the step
            const int j_hi = valid ? min(63, pos_r - key0) : -1;             // the keys this row sees: [j_lo, j_hi]
            const int j_lo = max(0, lo_r - key0);
            const bool whole = (kb_first + j) * KEYS + KEYS - 1 <= pos0 && (kb_first + j) * KEYS >= lo_last;
            float mx4[2] = {-INFINITY, -INFINITY};
            if (whole) {
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx4[e & 1] = fmaxf(mx4[e & 1], __uint_as_float(sv[q2][e]));
            } else {
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int jj = q2 * 32 + e;
                        if (jj >= j_lo && jj <= j_hi) mx4[e & 1] = fmaxf(mx4[e & 1], __uint_as_float(sv[q2][e]));
                    }
            }
            // the row's max: the two threads of a row exchange theirs through shared memory (two buffers in turn: a
            // buffer is written again only after the barrier of the step between, which both pass after reading it)
            const int buf = (j & 1) * 2 * ROWS;
            my_x[buf] = fmaxf(mx4[0], mx4[1]);
            // the barrier also carries the "a wait ran out somewhere" flag as a reduction, so that all 256 threads of
            // the tile leave together (a flag another warp sets while some threads are past their own look at it
            // would otherwise split them, and the next barrier would never fill)
            int any_bad;
            {
                const int bad = *gave_up;
                asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 q, %2, 0;\nbar.red.or.pred p, %1, 256, q;\nselp.b32 %0, 1, 0, p;\n}"
                             : "=r"(any_bad) : "r"(1 + x), "r"(bad) : "memory");
            }
            if (any_bad) { ok = false; break; }
            const float m_row = fmaxf(my_x[buf], other_x[buf]) * sl2;       // sl2 > 0: the max commutes with the scaling
            // the max in use stays unless it would be exceeded by more than PP_GROW somewhere in the warp
            float m_new, corr = 1.f;
            if (j == 0) {
                m_new = m_row;
            } else {
                const bool grow = m_row > m_used + PP_GROW;                  // (true for m_used = -inf and a finite m_row)
                const bool rescale = __any_sync(0xffffffffu, grow);
                m_new = grow ? m_row : m_used;
                corr = (m_used == -INFINITY) ? 0.f : ex2(m_used - m_new);   // 1 when the max stays
                if (!mbar_wait(&o_done[x], (j - 1) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 47, j, r); *gave_up = 1; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (rescale) {                                              // this thread's dims of the accumulated output, in place
#pragma unroll 1
                    for (int c = 0; c < HD / 2; c += 16) {
                        float ov[16];
                        tmem_ld16(t_o + c, ov);
                        uint32_t ow[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) ow[e] = __float_as_uint(ov[e] * corr);
                        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                                     ::"r"(t_o + c), "r"(ow[0]), "r"(ow[1]), "r"(ow[2]), "r"(ow[3]), "r"(ow[4]), "r"(ow[5]), "r"(ow[6]), "r"(ow[7]),
                                       "r"(ow[8]), "r"(ow[9]), "r"(ow[10]), "r"(ow[11]), "r"(ow[12]), "r"(ow[13]), "r"(ow[14]), "r"(ow[15]) : "memory");
                    }
                    tmem_wait_st();
                }
            }
            if (nB > 0 && (x == 1 || j > 0)) {
                // tile A's pass of step j goes before tile B's, B's before A's of step j + 1
                if (!mbar_wait(&turn[x], (x == 0 ? j - 1 : j) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 50, j, r); *gave_up = 1; }
            }
            const float nbase = (m_new == -INFINITY) ? 0.f : -m_new;
            float sum4[2] = {0.f, 0.f};
            auto exp_half = [&](const int q2) {             // keys 32 q2 .. 32 q2 + 31 of this thread's 64
                if (whole) {
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {         // 8 keys = one 16-byte chunk of P
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            const float p0 = ex2(fmaf(__uint_as_float(sv[q2][c8 * 8 + e]), sl2, nbase));
                            const float p1 = ex2(fmaf(__uint_as_float(sv[q2][c8 * 8 + e + 1]), sl2, nbase));
                            sum4[(e >> 1) & 1] += p0 + p1;
                            w[e >> 1] = pack2(p0, p1);
                        }
                        *reinterpret_cast<uint4*>(prow + (((q2 * 4 + c8) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            const int jj = q2 * 32 + c8 * 8 + e;
                            const float p0 = (jj >= j_lo && jj <= j_hi) ? ex2(fmaf(__uint_as_float(sv[q2][c8 * 8 + e]), sl2, nbase)) : 0.f;
                            const float p1 = (jj + 1 >= j_lo && jj + 1 <= j_hi) ? ex2(fmaf(__uint_as_float(sv[q2][c8 * 8 + e + 1]), sl2, nbase)) : 0.f;
                            sum4[(e >> 1) & 1] += p0 + p1;
                            w[e >> 1] = pack2(p0, p1);
                        }
                        *reinterpret_cast<uint4*>(prow + (((q2 * 4 + c8) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            };
            exp_half(0);
            // each thread's first 32 keys' probabilities are in shared memory (and the output is scaled): their share of P V may run
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&p_half[x]);
            // the other tile may begin its pass when this one is half way through its own: one tile's pass alone keeps
            // the exp2 units at about 70%, two whole passes at once take twice as long each
            if (nB > 0) mbar_arrive(&turn[x ^ 1]);
            exp_half(1);
            l_run = l_run * corr + (sum4[0] + sum4[1]);
            m_used = m_new;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&p_ready[x]);
        }
        if (x == 0 && nB > nA) {
            // Tile B's one step more has no pass of A's to wait for: A gives it its turn.  But only once B has taken the
            // turn before (B's arrival of step nA - 1, the one a step nA of A's would wait for): two arrivals of A's in a
            // row could otherwise complete two phases before B has looked at the first, and a wait by parity cannot tell
            // "two on" from "not yet".
            if (!mbar_wait(&turn[0], (nA - 1) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 50, nA, r); *gave_up = 1; }
            mbar_arrive(&turn[1]);
        }
        if (ok && n_x > 0) {
            if (!mbar_wait(&o_done[x], (n_x - 1) & 1)) { report(a.status, IMPARO_ST_WAIT_LIMIT, 48, n_x, r); *gave_up = 1; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the row's sum: the two threads' shares, in the order (keys 0-63, keys 64-127)
            const int buf = (n_x & 1) * 2 * ROWS;
            my_x[buf] = l_run;
            asm volatile("bar.sync %0, 256;" ::"r"(1 + x) : "memory");
            const float l = half == 0 ? my_x[buf] + other_x[buf] : other_x[buf] + my_x[buf];
            if (!*gave_up) {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                uint32_t ov[32];
                tmem_ld32_nowait(t_o, ov);
                tmem_wait_ld();
                keep32(ov);
                if (valid) {
                    uint4* dst = reinterpret_cast<uint4*>(a.out + row_off + half * (HD / 2));
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        dst[q] = make_uint4(pack2(__uint_as_float(ov[q * 8]) * inv, __uint_as_float(ov[q * 8 + 1]) * inv),
                                            pack2(__uint_as_float(ov[q * 8 + 2]) * inv, __uint_as_float(ov[q * 8 + 3]) * inv),
                                            pack2(__uint_as_float(ov[q * 8 + 4]) * inv, __uint_as_float(ov[q * 8 + 5]) * inv),
                                            pack2(__uint_as_float(ov[q * 8 + 6]) * inv, __uint_as_float(ov[q * 8 + 7]) * inv));
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

static int launch_pp(const CUtensorMap& mk, const CUtensorMap& mv, const Args& a, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = 1024 + 2 * REGION + 4 * REGION + (size_t)PP_STAGES * 2 * REGION + 256 + 2 * 2 * 2 * ROWS * 4;
    static bool configured = false;
    cudaError_t e;
    if (!configured) {
        e = cudaFuncSetAttribute(attn_prefill_pp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    e = launch(attn_prefill_pp_kernel, grid, dim3(PP_THREADS), smem, stream, mk, mv, a);
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace fa
}  // namespace imparo

using namespace imparo;

// bfloat16, head size 64 or 128, at most 8 query heads per kv head, pages of 16, 32, 64 or 128
// positions; else -8 (the caller uses another kernel).  mode bit 0: at head size 64 the kernel that gives a CTA two
// query tiles in turn (else, and at head size 128, one tile per CTA); bit 1: the kernel lets its dependents come only
// after its own wait, for a next kernel that runs beside it (imparo_attention_decode_mma with overlap_prev).
// n_tok is the batch's token count, n_items its requests.  The caches are [n_pages * page_size rows, nkv * hd] arenas.
extern "C" int imparo_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache,
                                           const int* item_row_start, const int* item_start_pos, int n_items,
                                           const int* table, int max_blocks, int page_size, int n_pages,
                                           int window, float scale, void* out, int n_tok, int nh, int nkv, int hd,
                                           int mode, int* status, cudaStream_t stream) {
    const int two_tiles = mode & 1;
    if (n_tok <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0) return -5;
    const int G = nh / nkv;
    if (G > 8 || (hd != 64 && hd != 128)) return -8;
    if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return -8;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return -8;
    if (!(scale > 0.f)) return -8;                           // the row max is taken before the scaling
    const int TQ = fa::ROWS / G;
    const long long tiles = (n_tok + TQ - 1) / TQ + n_items;          // an upper bound: every request may end a tile early
    if (tiles > 65535) return -8;                            // the tiles are the grid's y extent: the caller uses another kernel
    CUtensorMap mk, mv;
    const uint64_t rows = (uint64_t)n_pages * page_size, cols = (uint64_t)nkv * hd;
    int rc = tc::get_map(k_cache, rows, cols, cols, (uint32_t)page_size, &mk);
    if (rc) return rc;
    rc = tc::get_map(v_cache, rows, cols, cols, (uint32_t)page_size, &mv);
    if (rc) return rc;
    fa::Args a;
    a.q = (const __nv_bfloat16*)q; a.out = (__nv_bfloat16*)out;
    a.item_row_start = item_row_start; a.item_start_pos = item_start_pos; a.table = table; a.status = status;
    a.n_items = n_items; a.max_blocks = max_blocks; a.page_size = page_size; a.n_pages = n_pages; a.window = window;
    a.nh = nh; a.nkv = nkv; a.scale = scale;
    a.late_trigger = (mode >> 1) & 1;
    if (hd == 64 && two_tiles) {
        // two tiles per CTA: half as many CTAs along y (an upper bound again)
        const long long pairs = (n_tok + 2 * TQ - 1) / (2 * TQ) + n_items;
        return fa::launch_pp(mk, mv, a, dim3(nkv, (unsigned)pairs), stream);
    }
    dim3 grid(nkv, (unsigned)tiles);
    return hd == 64 ? fa::launch_tc<64>(mk, mv, a, grid, stream) : fa::launch_tc<128>(mk, mv, a, grid, stream);
}
