// bfloat16 matrix product on the 5th-generation tensor cores:
//     out[T, N] (+)= X[T, K] * W[N, K]^T        (both operands K-major, 32-bit accumulation)
//
// The weight tile is the MMA's M operand (128 rows of W per CTA) and the tokens are its N
// operand (16..256 tokens per CTA), so a decode step of a few tokens still fills the
// 128-row instruction and the kernel's job is to stream W from HBM once: TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast) fills a ring of shared-memory
// stages, one elected thread issues tcgen05.mma with the accumulator in tensor memory,
// tcgen05.commit hands stages back to the producer, and four warps read the accumulator with
// tcgen05.ld and write out[token, n] (32 lanes = 32 consecutive n: coalesced).
//
// Few output tiles (N small) are cut along K as well (split-K): the splits of one tile are the
// CTAs of one thread-block cluster.  Each leaves its partial tile in its own shared memory;
// after a cluster barrier every CTA folds a share of the tile's tokens, reading the partials
// of all splits through distributed shared memory in split order, and runs the epilogue for
// them.  No global scratch, and the same sum every time.
//
// Epilogues: store bfloat16 | store float32 | add into float32 (the residual stream) |
// SwiGLU: the CTA's 128 rows are 64 gate rows and the 64 up rows of the same features,
// h = silu(gate) * up is written as bfloat16 [T, F]  (imparo-cpu/src/ops.rs:73-78;
// imparo-model/src/lfm2/workflow_cpu.rs:307-313).
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records
// IMPARO_ST_WAIT_LIMIT in the status word, stops waiting, frees its tensor memory and
// returns (the output of that launch is then garbage, and the host raises).
#include "tcgen05.cuh"

namespace imparo {
namespace tc {

constexpr int BM = 128;            // rows of W per CTA (MMA M)
constexpr int THREADS = 192;       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

enum Epilogue { STORE_BF16 = 0, STORE_F32 = 1, ADD_F32 = 2, SWIGLU_BF16 = 3, PARTIAL_F32 = 4 };
// Who makes the token operand.  PROD_NONE: it is a stored tensor, loaded by TMA beside the W tiles.  Otherwise
// the four epilogue warps (idle during the main loop) compute it after the wait on the previous kernel and write
// it, as bfloat16 in the MMA's swizzled K-major layout, into shared memory for all k-blocks of this CTA; the ring
// then carries W tiles only, and the kernel that would have made the tensor is gone from the chain:
//   PROD_COMBINE  the ordered combine of the split-key attention's partial results
enum Producer { PROD_NONE = 0, PROD_COMBINE = 3 };

template <int EPI>
__device__ __forceinline__ void store_out(void* out, size_t o, float v) {
    if (EPI == STORE_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
    else if (EPI == STORE_F32) reinterpret_cast<float*>(out)[o] = v;
    else reinterpret_cast<float*>(out)[o] += v;
}

struct Params {
    void* out;               // [T, ldo]
    float* scratch;          // split-K partials [splits][T][N]
    int* counters;           // one per (token tile, row tile); zero before the launch, zero after
    int* status;
    int T, N, K, ldo;        // N = rows of W (for SWIGLU: F, W has 2F rows)
    int splits, kblocks;     // kblocks = ceil(K / BK)
    int kb_cap;                  // PROD != NONE: k-blocks of the resident token operand (the most one split owns)
    int tma_out;                 // PARTIAL_F32: the partial tile leaves through shared memory and one TMA store (map_o)
    // PROD_COMBINE: token operand [t, h * hd + d] = sum_s acc[t,h,s,d] f_s / sum_s l_s f_s, f_s = exp(m_s - max m)
    const float* cb_acc;         // [T, heads, splits, hd]
    const float* cb_ml;          // [T, heads, splits, 2]  (max, sum)
    int cb_splits, cb_hd, cb_heads;
};

__device__ __forceinline__ uint4 pack8(const float* v) {
    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
    return make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                      *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
}
// shared memory: [stages] x (A tile 16 KB | B tile NT*128 B), then barriers; the exchange buffer of the
// SwiGLU epilogue lies over the ring's first stage.  Tiles are 1024-byte aligned (128-byte swizzle).  With a producer
// (PROD != PROD_NONE) the ring carries W tiles only and the token operand of all the CTA's k-blocks
// follows the ring.
template <int PROD> struct ThreadsOf { static constexpr int value = (PROD == PROD_COMBINE) ? 320 : THREADS; };

template <int NT, int STAGES, int EPI, int PROD>
__global__ void __launch_bounds__(ThreadsOf<PROD>::value, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
            const __grid_constant__ CUtensorMap map_o, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = NT * BK * 2, STAGE_BYTES = PROD != PROD_NONE ? A_BYTES : A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = NT < 32 ? 32 : NT;
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* bres = smem + STAGES * STAGE_BYTES;                               // PROD: [kb_cap][NT][128 B]
    uint8_t* aux = bres + (PROD != PROD_NONE ? (size_t)p.kb_cap * B_BYTES : 0);
    uint64_t* full = reinterpret_cast<uint64_t*>(aux);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint64_t* b_ready = acc_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_ready + 1);
    int* flags = reinterpret_cast<int*>(tmem_slot + 1);            // [0]: this CTA folds the splits
    // SwiGLU: 2 x [128][17], a 16-token chunk each.  The epilogue runs when every product has read its stage and
    // no load is in flight, so the exchange buffer lies over the ring's first stage and costs no shared memory of
    // its own: what it would have taken is a deeper ring, or room for the next kernel's CTA beside this one.
    float* exch = reinterpret_cast<float*>(smem);
    static_assert(EPI != SWIGLU_BF16 || STAGES * STAGE_BYTES >= 2 * 128 * 17 * 4, "the exchange buffer lies over the ring");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x;                 // which 128 rows of W (SwiGLU: which 64 features)
    const int tile_t = blockIdx.y;                 // which NT tokens
    int split = blockIdx.z;                        // with split-K: this CTA's rank in its cluster
    // PARTIAL_F32: the splits are plain CTAs (blockIdx.z), each stores its partial tile and is done
    const bool clustered = EPI != PARTIAL_F32 && p.splits > 1;
    if (clustered) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(split));
    const int kb_begin = (int)(((long long)p.kblocks * split) / p.splits);
    const int kb_end = (int)(((long long)p.kblocks * (split + 1)) / p.splits);
    const int n_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        mbar_init(b_ready, (PROD == PROD_COMBINE) ? 256 : 128);
        flags[0] = 0;
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
        if (lane == 0) {
            // Weights are written by no kernel: the first ring of W tiles is requested before
            // waiting for the previous kernel, so it streams in while that kernel finishes.
            auto load_w = [&](int i) {
                const int s = i % STAGES;
                uint8_t* a = smem + s * STAGE_BYTES;
                mbar_expect_tx(&full[s], STAGE_BYTES);          // PROD: the W tile only
                const int k0 = (kb_begin + i) * BK;
                if (EPI == SWIGLU_BF16) {
                    tma_load_2d(a, &map_w, &full[s], k0, tile_n * 64);                       // 64 gate rows
                    tma_load_2d(a + A_BYTES / 2, &map_w, &full[s], k0, p.N + tile_n * 64);   // their 64 up rows
                } else {
                    tma_load_2d(a, &map_w, &full[s], k0, tile_n * BM);
                }
            };
            auto load_x = [&](int i) {
                if (PROD != PROD_NONE) return;                   // the input rows are made in place by the epilogue warps
                const int s = i % STAGES;
                tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, &map_x, &full[s], (kb_begin + i) * BK, tile_t * NT);
            };
            const int early = n_kb < STAGES ? n_kb : STAGES;
            pdl_trigger();
            for (int i = 0; i < early; ++i) load_w(i);
            pdl_wait();                                          // (PROD: nothing below needs it; it orders this thread's stamps)
            for (int i = 0; i < early; ++i) load_x(i);
            for (int i = early; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&empty[s], ((i / STAGES) - 1) & 1)) {
                    report(p.status, IMPARO_ST_WAIT_LIMIT, 10, i, s);
                    break;
                }
                load_w(i);
                load_x(i);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(BM, NT);
            bool ok = true;
            if (PROD != PROD_NONE && !mbar_wait(b_ready, 0)) {
                report(p.status, IMPARO_ST_WAIT_LIMIT, 13, tile_n, split);
                ok = false;
            }
            if (PROD == PROD_COMBINE) timeline_mark(0);       // the token operand is made
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&full[s], (i / STAGES) & 1)) {
                    report(p.status, IMPARO_ST_WAIT_LIMIT, 11, i, s);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                const uint32_t b_addr = PROD != PROD_NONE ? smem_u32(bres + (size_t)i * B_BYTES) : a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // 16 elements along K = 32 bytes inside the 128-byte swizzle atom
                    umma(tmem_base, smem_desc(a_addr + k * UMMA_K * 2), smem_desc(b_addr + k * UMMA_K * 2), idesc,
                         (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);        // the stage is free once these MMAs have read it
            }
            umma_commit(acc_ready);            // arrives when every MMA issued above is complete
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +32 ----
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                       // row of the CTA's W tile
        pdl_wait();                                             // before any global write or residual read
        if (PROD == PROD_COMBINE) {
            // A thread per (live token row of the tile, 16-byte chunk = 8 consecutive k) of this CTA's k-range; eight
            // warps (2..9) share the items.  The (max, sum) pairs of an item and the first accumulators are requested
            // together, so that the usual case costs two round trips to memory.
            const int pe = (int)threadIdx.x - 64;                               // 0 .. 255
            const int k_lo = kb_begin * BK, k_hi = min(p.K, kb_end * BK);
            const int chunks = n_kb * (BK / 8);
            const int live = min(NT, p.T - tile_t * NT);
            const int n_items = live * chunks;
            for (int item = pe; item < NT * chunks; item += 256) {
                const int r = item / chunks, cc = item - r * chunks;
                const int k = k_lo + cc * 8;
                const int t = tile_t * NT + r;
                float yv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) yv[i] = 0.f;
                if (item < n_items && k < k_hi) {                             // K is a multiple of 8: whole chunks only
                    {
                        const int hd = p.cb_hd, S = p.cb_splits;
                        const int h = k / hd, d = k - h * hd;
                        const size_t th = (size_t)t * p.cb_heads + h;
                        const float2* ml = reinterpret_cast<const float2*>(p.cb_ml) + th * S;
                        const float* acc_p = p.cb_acc + th * S * hd + d;
                        float L = 0.f;
                        if (S <= 16) {
                            // the (max, sum) pairs and the first eight splits' accumulators are requested together
                            float2 v[16];
                            float4 a[8][2];
#pragma unroll
                            for (int u = 0; u < 16; ++u) v[u] = u < S ? __ldcg(ml + u) : make_float2(-INFINITY, 0.f);
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                if (u < S) {
                                    a[u][0] = __ldcg(reinterpret_cast<const float4*>(acc_p + (size_t)u * hd));
                                    a[u][1] = __ldcg(reinterpret_cast<const float4*>(acc_p + (size_t)u * hd + 4));
                                }
                            }
                            float M = -INFINITY;
#pragma unroll
                            for (int u = 0; u < 16; ++u) if (v[u].y > 0.f) M = fmaxf(M, v[u].x);
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                if (half == 1) {
#pragma unroll
                                    for (int u = 0; u < 8; ++u) {
                                        if (8 + u < S) {
                                            a[u][0] = __ldcg(reinterpret_cast<const float4*>(acc_p + (size_t)(8 + u) * hd));
                                            a[u][1] = __ldcg(reinterpret_cast<const float4*>(acc_p + (size_t)(8 + u) * hd + 4));
                                        }
                                    }
                                }
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    const int sidx = half * 8 + u;
                                    float2 vv = v[0];
#pragma unroll
                                    for (int q = 1; q < 16; ++q) if (q == sidx) vv = v[q];
                                    if (sidx < S && vv.y > 0.f) {
                                        const float f = expf(vv.x - M);
                                        yv[0] += a[u][0].x * f; yv[1] += a[u][0].y * f; yv[2] += a[u][0].z * f; yv[3] += a[u][0].w * f;
                                        yv[4] += a[u][1].x * f; yv[5] += a[u][1].y * f; yv[6] += a[u][1].z * f; yv[7] += a[u][1].w * f;
                                        L += vv.y * f;
                                    }
                                }
                            }
                        } else {
                            float M = -INFINITY;
                            for (int s0 = 0; s0 < S; ++s0) { const float2 v = __ldcg(ml + s0); if (v.y > 0.f) M = fmaxf(M, v.x); }
                            for (int s0 = 0; s0 < S; s0 += 4) {
                                float4 a[4], b[4];
                                float2 v[4];
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    if (s0 + u < S) {
                                        v[u] = __ldcg(ml + s0 + u);
                                        a[u] = __ldcg(reinterpret_cast<const float4*>(acc_p + (size_t)(s0 + u) * hd));
                                        b[u] = __ldcg(reinterpret_cast<const float4*>(acc_p + (size_t)(s0 + u) * hd + 4));
                                    }
                                }
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    if (s0 + u < S && v[u].y > 0.f) {
                                        const float f = expf(v[u].x - M);
                                        yv[0] += a[u].x * f; yv[1] += a[u].y * f; yv[2] += a[u].z * f; yv[3] += a[u].w * f;
                                        yv[4] += b[u].x * f; yv[5] += b[u].y * f; yv[6] += b[u].z * f; yv[7] += b[u].w * f;
                                        L += v[u].y * f;
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) yv[i] = L > 0.f ? yv[i] / L : 0.f;
                    }
                }
                const int i = cc / (BK / 8), chunk = cc % (BK / 8);
                *reinterpret_cast<uint4*>(bres + (size_t)i * B_BYTES + (size_t)r * 128 + ((chunk ^ (r & 7)) << 4)) = pack8(yv);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b_ready)) : "memory");
            if (warp >= 6) goto done;                                           // warps 6..9 only help to make the operand
        }
        bool ok = n_kb == 0 || mbar_wait(acc_ready, 0);
        if (threadIdx.x == 64 && PROD != PROD_COMBINE) timeline_mark(0);                // the accumulator is complete
        if (!ok && lane == 0) report(p.status, IMPARO_ST_WAIT_LIMIT, 12, tile_n, split);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int t0 = tile_t * NT;
        constexpr int CH = NT >= 64 ? 4 : NT / 16;              // accumulator chunks fetched per wait

        if (EPI == SWIGLU_BF16) {
            // rows 0..63 hold gate, rows 64..127 hold up of features tile_n*64 + (row % 64).  Both go
            // through shared memory, and the 128 threads then share the (feature, token) pairs: a
            // lone warp doing sixteen silus in a row is bound by instruction latency
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
            const int e = (int)threadIdx.x - 64;
            const int ff = e & 63, parity = e >> 6;
            const int f = tile_n * 64 + ff;
#pragma unroll 1
            for (int c = 0; c < NT; c += 16 * CH) {
                float v[CH][16];
                tmem_ld_chunks<CH>(taddr + c, v);
#pragma unroll
                for (int u = 0; u < CH; ++u) {
                    // two exchange buffers in turn: one barrier per 16 tokens (a buffer is rewritten only
                    // after the barrier of the chunk between, which every thread passes after reading it)
                    float* ex = exch + (u & 1) * (128 * 17);
#pragma unroll
                    for (int j = 0; j < 16; ++j) ex[row * 17 + j] = v[u][j];
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (f < p.N) {
#pragma unroll
                        for (int j = 0; j < 16; j += 2) {
                            const int t = t0 + c + 16 * u + j + parity;
                            if (t < p.T)
                                out[(size_t)t * p.ldo + f] = __float2bfloat16_rn(silu_bf16(ex[ff * 17 + j + parity]) * ex[(64 + ff) * 17 + j + parity]);
                        }
                    }
                }
                if (CH == 1 || c + 16 * CH < NT) asm volatile("bar.sync 1, 128;" ::: "memory");
            }
        } else {
            const int n = tile_n * BM + row;
            if (EPI == PARTIAL_F32) {
                // this split's partial tile -> scratch[split][token][n]; whoever reads the stream next
                // adds the splits in order (rows.cu: add_partials_rmsnorm)
                float* part = p.scratch + (size_t)split * p.T * p.N;
                if (p.tma_out) {
                    // Through shared memory (the stage ring is idle now) as [token][row] and out with ONE store of
                    // the TMA engine: a thread's 16 to 64 strided 32-bit stores took the load/store unit 0.4 to 2.4 us
                    // at the very end of the kernel, where the next kernel waits for it.  Rows and tokens beyond the
                    // tensor are clipped by the engine.
                    float* stage = reinterpret_cast<float*>(smem);
#pragma unroll 1
                    for (int c = 0; c < NT; c += 16 * CH) {
                        float v[CH][16];
                        tmem_ld_chunks<CH>(taddr + c, v);
#pragma unroll
                        for (int u = 0; u < CH; ++u)
#pragma unroll
                            for (int j = 0; j < 16; ++j) stage[(c + 16 * u + j) * BM + row] = v[u][j];
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (threadIdx.x == 64) {
                        tma_store_3d(&map_o, stage, tile_n * BM, t0, split);
                        tma_store_wait_read();
                    }
                } else
#pragma unroll 1
                for (int c = 0; c < NT; c += 16 * CH) {
                    float v[CH][16];
                    tmem_ld_chunks<CH>(taddr + c, v);
                    if (n < p.N) {
#pragma unroll
                        for (int u = 0; u < CH; ++u)
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int t = t0 + c + 16 * u + j;
                                if (t < p.T) part[(size_t)t * p.N + n] = v[u][j];
                            }
                    }
                }
            } else if (p.splits == 1) {
#pragma unroll 1
                for (int c = 0; c < NT; c += 16) {
                    float v[16];
                    tmem_ld16(taddr + c, v);
                    if (n < p.N) {
                        if (EPI == ADD_F32) {
                            // all sixteen reads of the stream before any write: the compiler must not
                            // chain load-add-store sixteen times (it cannot prove the addresses differ)
                            float old[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int t = t0 + c + j;
                                old[j] = t < p.T ? reinterpret_cast<const float*>(p.out)[(size_t)t * p.ldo + n] : 0.f;
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int t = t0 + c + j;
                                if (t < p.T) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = old[j] + v[j];
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int t = t0 + c + j;
                                if (t < p.T) store_out<EPI>(p.out, (size_t)t * p.ldo + n, v[j]);
                            }
                        }
                    }
                }
            } else {
                // this split's partial tile -> own shared memory, [token][row] (the stage ring is idle now)
                float* part = reinterpret_cast<float*>(smem);
#pragma unroll 1
                for (int c = 0; c < NT; c += 16) {
                    float v[16];
                    tmem_ld16(taddr + c, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) part[(c + j) * BM + row] = v[j];
                }
            }
        }
    }
done:
    if (clustered) {
        // every thread of every CTA of the cluster: partials are written / may be read
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2 && warp < 6) {
            const int quad = warp & 3;
            const int row = quad * 32 + lane;
            const int n = tile_n * BM + row;
            const int t0 = tile_t * NT;
            const uint32_t my = smem_u32(smem) + (uint32_t)row * 4;
            // CTA `split` folds token columns split, split + splits, ...: the sum runs over the
            // splits in order 0, 1, 2, ... whichever CTA does it
            for (int c = split; c < NT; c += p.splits) {
                const int t = t0 + c;
                if (t >= p.T) break;
                float acc = 0.f;
                for (int s0 = 0; s0 < p.splits; s0 += 8) {            // eight remote loads in flight, adds in split order
                    float v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        v[u] = 0.f;
                        if (s0 + u < p.splits) {
                            uint32_t remote;
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(my + (uint32_t)c * BM * 4), "r"(s0 + u));
                            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[u]) : "r"(remote));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (s0 + u < p.splits) acc += v[u];
                }
                if (n < p.N) store_out<EPI>(p.out, (size_t)t * p.ldo + n, acc);
            }
        }
        // nobody leaves while its shared memory may still be read
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) timeline_mark(1);                     // this CTA's epilogue is done
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------
// imparo_gemm_tc_configure() walks every instantiation once with this set: the shared-memory attribute of each is
// set and nothing is launched.  The runtime refuses that call (and the occupancy query of the cluster plan) while a
// stream is being captured, so an engine that records its steps into graphs does it beforehand.
static thread_local bool g_configure_only = false;

template <int NT, int STAGES, int EPI, int PROD = PROD_NONE>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, const Params& p, dim3 grid, cudaStream_t stream) {
    constexpr size_t fixed = 1024 + (size_t)STAGES * (BM * BK * 2 + (PROD != PROD_NONE ? 0 : NT * BK * 2)) + 256;
    static_assert(fixed <= 227 * 1024, "stage ring exceeds shared memory");
    const size_t smem = fixed + (PROD != PROD_NONE ? (size_t)p.kb_cap * NT * BK * 2 : 0);
    if (smem > 227 * 1024) return -25;          // the resident input does not fit: the caller makes the tensor with its own kernel
    auto kern = gemm_kernel<NT, STAGES, EPI, PROD>;
    static size_t configured = 0;               // per instantiation: the largest size asked for so far
    cudaError_t e;
    if (smem > configured) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    if (g_configure_only) return 0;
    e = timeline_note(reinterpret_cast<const void*>(kern));
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ThreadsOf<PROD>::value);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = EPI == PARTIAL_F32 ? 1 : grid.z;     // the splits of a tile are one cluster
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = imparo_pdl_enabled() ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kern, mw, mx, mo, p);
    return e == cudaSuccess ? 0 : (int)e;
}

// How many clusters of `cluster` CTAs of this kernel the device holds at once (0 on error).
template <int NT, int STAGES, int EPI>
static int max_clusters(int cluster) {
    constexpr size_t smem = 1024 + (size_t)STAGES * (BM * BK * 2 + NT * BK * 2) + 256;
    auto kern = gemm_kernel<NT, STAGES, EPI, PROD_NONE>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, cluster);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = cluster;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

// Ring depth.  Measured in the decode step (batch 8): 11 stages 1.050 ms, 5 stages 1.038 ms,
// 3 stages 1.076 ms.  A ring of 5 leaves room for a second CTA per SM, and with programmatic
// dependent launch that second CTA is the NEXT product's: it fills its ring with weights while
// this one is still streaming, which is worth more than a deeper ring of one's own.  (Again later, at 0.77 ms
// per step: 4 stages 0.788 ms, 5 stages 0.764, 6 stages 0.767.)
constexpr int deep_stages_for(int nt) { return nt <= 32 ? 5 : nt <= 64 ? 4 : nt == 128 ? 5 : 4; }
constexpr int stages_for(int nt) { return nt <= 64 ? 4 : nt == 128 ? 5 : 4; }
// The SwiGLU product (gate+up, the step's largest stream, K whole in every CTA) takes one stage more than would
// fit with an exchange buffer of its own; the buffer lies over the ring instead.  Batch 8: 5 stages 0.769-0.773 ms per
// step, 6 stages 0.763-0.765, 7 stages 0.781-0.784 (the next product's CTA no longer fits beside it).  Batch 64:
// 4 stages 1.272-1.284 ms, 5 stages 1.236-1.242, 6 stages 1.233-1.236.
constexpr int swiglu_stages_for(int nt) { return nt <= 64 ? 6 : nt == 128 ? 5 : 4; }

template <int EPI>
static int launch_nt(int nt, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, const Params& p, dim3 grid, cudaStream_t stream) {
    const bool deep = (long long)grid.x * grid.y * grid.z <= 148;
    if (EPI == SWIGLU_BF16) {
        switch (nt) {
            case 16: return launch<16, swiglu_stages_for(16), EPI>(mw, mx, mo, p, grid, stream);
            case 32: return launch<32, swiglu_stages_for(32), EPI>(mw, mx, mo, p, grid, stream);
            case 64: return launch<64, swiglu_stages_for(64), EPI>(mw, mx, mo, p, grid, stream);
            case 128: return launch<128, swiglu_stages_for(128), EPI>(mw, mx, mo, p, grid, stream);
            case 256: return launch<256, swiglu_stages_for(256), EPI>(mw, mx, mo, p, grid, stream);
        }
        return -22;
    }
    switch (nt) {
        case 16: return deep ? launch<16, deep_stages_for(16), EPI>(mw, mx, mo, p, grid, stream) : launch<16, stages_for(16), EPI>(mw, mx, mo, p, grid, stream);
        case 32: return deep ? launch<32, deep_stages_for(32), EPI>(mw, mx, mo, p, grid, stream) : launch<32, stages_for(32), EPI>(mw, mx, mo, p, grid, stream);
        case 64: return deep ? launch<64, deep_stages_for(64), EPI>(mw, mx, mo, p, grid, stream) : launch<64, stages_for(64), EPI>(mw, mx, mo, p, grid, stream);
        case 128: return deep ? launch<128, deep_stages_for(128), EPI>(mw, mx, mo, p, grid, stream) : launch<128, stages_for(128), EPI>(mw, mx, mo, p, grid, stream);
        case 256: return launch<256, stages_for(256), EPI>(mw, mx, mo, p, grid, stream);
    }
    return -22;
}

// resident clusters by (token tile, cluster size), asked of the runtime once
static int resident_clusters(int nt, int cluster) {
    static int table[5][9];
    static bool known[5][9];
    const int i = nt == 16 ? 0 : nt == 32 ? 1 : nt == 64 ? 2 : nt == 128 ? 3 : 4;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!known[i][cluster]) {
        int n = 0;
        switch (nt) {
            case 16: n = max_clusters<16, deep_stages_for(16), ADD_F32>(cluster); break;
            case 32: n = max_clusters<32, deep_stages_for(32), ADD_F32>(cluster); break;
            case 64: n = max_clusters<64, deep_stages_for(64), ADD_F32>(cluster); break;
            case 128: n = max_clusters<128, deep_stages_for(128), ADD_F32>(cluster); break;
            default: n = max_clusters<256, stages_for(256), ADD_F32>(cluster); break;
        }
        table[i][cluster] = n;
        known[i][cluster] = true;
    }
    return table[i][cluster];
}

}  // namespace tc
}  // namespace imparo

using namespace imparo::tc;

extern "C" int imparo_gemm_tc_max_clusters(int nt, int cluster) {
    if (cluster < 1 || cluster > 8) return -1;
    return resident_clusters(nt, cluster);
}

// How the launcher would cut a product: token tile, splits along K, scratch floats and
// counters it needs.  epilogue: 0 store bf16, 1 store f32, 2 add f32, 3 SwiGLU (N = F).
extern "C" int imparo_gemm_tc_plan(int T, int N, int K, int epilogue, int* token_tile, int* splits,
                                   long long* scratch_floats, int* n_counters) {
    if (T <= 0 || N <= 0 || K <= 0) return -2;
    const int nt = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
    const int row_tiles = epilogue == SWIGLU_BF16 ? (N + 63) / 64 : (N + BM - 1) / BM;
    const int tok_tiles = (T + nt - 1) / nt;
    const int kblocks = (K + BK - 1) / BK;
    int s = 1;
    if (epilogue == PARTIAL_F32) {
        // plain CTAs, no cluster: as many splits as fill the device once, at least 4 k-blocks each
        const int tiles = row_tiles * tok_tiles;
        s = tiles >= 148 ? 1 : 148 / tiles;
        if (s > kblocks / 4) s = kblocks / 4;
        if (s < 1) s = 1;
        if (s > 16) s = 16;
    } else if (epilogue != SWIGLU_BF16) {
        // The splits of a tile are one cluster (at most 8 CTAs, the portable size).  Take the
        // cluster size that puts the most CTAs on the device in ONE wave: all the tiles'
        // clusters must be resident together.  Never cut K below 4 blocks per split.
        const int tiles = row_tiles * tok_tiles;
        int best = 1;
        if (tiles < 120) {
            for (int c = 2; c <= 8 && c <= kblocks / 4; ++c)
                if (tiles <= resident_clusters(nt, c) && tiles * c > tiles * best) best = c;
        }
        s = best;
    }
    *token_tile = nt;
    *splits = s;
    *scratch_floats = epilogue == PARTIAL_F32 ? (long long)s * T * N : 0;   // else partials live in the cluster's shared memory
    *n_counters = 0;
    return 0;
}

// The split partials leave by a TMA store where the rows are 16 bytes wide and aligned (N a multiple of 4) and the
// token tile is at most 64 (the staged tile must fit the idle stage ring); else by plain stores.
static int partials_map(float* scratch, int T, int N, int splits, int nt, Params& p, CUtensorMap& mo) {
    p.tma_out = 0;
    if (N % 4 != 0 || (((uintptr_t)scratch) & 15) || nt > 64) return 0;
    int rc = get_map_partials(scratch, (uint64_t)N, (uint64_t)T, (uint64_t)splits, (uint32_t)nt, &mo);
    if (rc) return rc;
    p.tma_out = 1;
    return 0;
}

// x: [T, K] bfloat16 with row stride ldx (elements), inside a buffer of x_rows_alloc rows.
// w: [N, K] bfloat16 dense (SwiGLU: [2N, K], gate rows then up rows).  out: [T, ldo].
// scratch / counters: from imparo_gemm_tc_plan; counters must be zero (they are left zero).
extern "C" int imparo_gemm_tc(const void* x, int ldx, int x_rows_alloc, const void* w, void* out, int ldo,
                              int T, int N, int K, int epilogue, float* scratch, int* counters, int* status,
                              cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0) return -23;                   // TMA: 16-byte rows
    if (((uintptr_t)x | (uintptr_t)w) & 15) return -23;
    int nt, splits, ncnt;
    long long sfl;
    imparo_gemm_tc_plan(T, N, K, epilogue, &nt, &splits, &sfl, &ncnt);
    const int w_rows = epilogue == SWIGLU_BF16 ? 2 * N : N;
    CUtensorMap mw, mx;
    int rc = get_map(w, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, epilogue == SWIGLU_BF16 ? 64u : (uint32_t)BM, &mw);
    if (rc) return rc;
    rc = get_map(x, (uint64_t)(x_rows_alloc > T ? x_rows_alloc : T), (uint64_t)K, (uint64_t)ldx, (uint32_t)nt, &mx);
    if (rc) return rc;
    Params p = {};
    p.out = out; p.scratch = scratch; p.counters = counters; p.status = status;
    p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.splits = splits; p.kblocks = (K + BK - 1) / BK;
    const int row_tiles = epilogue == SWIGLU_BF16 ? (N + 63) / 64 : (N + BM - 1) / BM;
    dim3 grid(row_tiles, (T + nt - 1) / nt, splits);
    if (grid.y > 65535) return -2;
    CUtensorMap mo = mw;                                                    // unused unless the partials leave by TMA
    switch (epilogue) {
        case STORE_BF16: return launch_nt<STORE_BF16>(nt, mw, mx, mo, p, grid, stream);
        case STORE_F32: return launch_nt<STORE_F32>(nt, mw, mx, mo, p, grid, stream);
        case ADD_F32: return launch_nt<ADD_F32>(nt, mw, mx, mo, p, grid, stream);
        case SWIGLU_BF16: return launch_nt<SWIGLU_BF16>(nt, mw, mx, mo, p, grid, stream);
        case PARTIAL_F32:
            if (!scratch) return -24;
            rc = partials_map(scratch, T, N, splits, nt, p, mo);
            if (rc) return rc;
            return launch_nt<PARTIAL_F32>(nt, mw, mx, mo, p, grid, stream);
    }
    return -22;
}


// ---- a product whose token operand the kernel makes itself: the attention's output product ----------------
// It takes out (32-bit stream, [T, N]) and either adds into it (epilogue 2) or leaves split partials in
// scratch (epilogue 4, scratch from imparo_gemm_tc_plan with that epilogue): the two forms the mixers' output
// products use.  T at most 16.  Returns -25 when it does not take the case.
static int launch_produced(int nt, int epilogue, const CUtensorMap& mw, const CUtensorMap& mo, const Params& p, dim3 grid, cudaStream_t stream) {
#define IMPARO_PRODUCED(NT_, ST_) \
    if (epilogue == PARTIAL_F32) return launch<NT_, ST_, PARTIAL_F32, PROD_COMBINE>(mw, mw, mo, p, grid, stream); \
    return launch<NT_, ST_, ADD_F32, PROD_COMBINE>(mw, mw, mo, p, grid, stream)
    // up to 16 tokens: with more, the eight producer warps walk several items each, one round trip after the other,
    // and the kernels apart are faster
    if (nt == 16) { IMPARO_PRODUCED(16, 6); }
#undef IMPARO_PRODUCED
    return -25;
}

static int produced_common(const void* w, float* out, int ldo, int T, int N, int K, int epilogue, float* scratch, int* status,
                           Params& p, CUtensorMap& mw, int& nt, dim3& grid) {
    if (K <= 0 || K % 8 != 0 || (((uintptr_t)w) & 15)) return -23;
    if (epilogue != ADD_F32 && epilogue != PARTIAL_F32) return -22;
    if (T > 16) return -25;
    int splits, ncnt;
    long long sfl;
    imparo_gemm_tc_plan(T, N, K, epilogue, &nt, &splits, &sfl, &ncnt);
    if (epilogue == PARTIAL_F32 && !scratch) return -24;
    int rc = get_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)BM, &mw);
    if (rc) return rc;
    p.out = out; p.scratch = scratch; p.status = status;
    p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.splits = splits; p.kblocks = (K + BK - 1) / BK;
    p.kb_cap = (p.kblocks + splits - 1) / splits;          // floor((s+1)k/S) - floor(sk/S) <= ceil(k/S)
    grid = dim3((N + BM - 1) / BM, (T + nt - 1) / nt, splits);
    return 0;
}

// out (+)= combine(partials) w^T: the ordered combine of the split-key attention (attention_split.cu) computed inside
// the output product.  part_acc [T, heads, splits, hd], part_ml [T, heads, splits, 2]; K = heads * hd.
extern "C" int imparo_gemm_tc_combine(const float* part_acc, const float* part_ml, int heads, int hd, int n_splits,
                                      const void* w, float* out, int ldo, int T, int N, int K, int epilogue, float* scratch,
                                      int* status, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (heads <= 0 || hd % 8 != 0 || heads * hd != K || n_splits < 1) return -2;
    if (n_splits > 64) return -25;
    if ((((uintptr_t)part_acc) | ((uintptr_t)part_ml)) & 15) return -23;
    Params p = {};
    CUtensorMap mw;
    int nt;
    dim3 grid;
    int rc = produced_common(w, out, ldo, T, N, K, epilogue, scratch, status, p, mw, nt, grid);
    if (rc) return rc;
    p.cb_acc = part_acc; p.cb_ml = part_ml; p.cb_splits = n_splits; p.cb_hd = hd; p.cb_heads = heads;
    CUtensorMap mo = mw;
    if (epilogue == PARTIAL_F32) {
        rc = partials_map(scratch, T, N, p.splits, nt, p, mo);
        if (rc) return rc;
    }
    return launch_produced(nt, epilogue, mw, mo, p, grid, stream);
}

// Every instantiation's shared-memory attribute and the cluster plan's occupancy table, ahead of the first launch
// (see g_configure_only).  Returns 0 or the first CUDA error.
extern "C" int imparo_gemm_tc_configure() {
    Params p = {};
    p.kb_cap = 1;
    CUtensorMap m = {};
    int rc = 0;
    g_configure_only = true;
    const int nts[5] = {16, 32, 64, 128, 256};
    for (int i = 0; i < 5 && rc == 0; ++i) {
        for (int deep = 0; deep < 2 && rc == 0; ++deep) {
            const dim3 grid(deep ? 1 : 1024, 1, 1);
            rc = launch_nt<STORE_BF16>(nts[i], m, m, m, p, grid, nullptr);
            if (!rc) rc = launch_nt<STORE_F32>(nts[i], m, m, m, p, grid, nullptr);
            if (!rc) rc = launch_nt<ADD_F32>(nts[i], m, m, m, p, grid, nullptr);
            if (!rc) rc = launch_nt<SWIGLU_BF16>(nts[i], m, m, m, p, grid, nullptr);
            if (!rc) rc = launch_nt<PARTIAL_F32>(nts[i], m, m, m, p, grid, nullptr);
        }
        for (int c = 2; c <= 8; ++c) resident_clusters(nts[i], c);
    }
    if (!rc) rc = launch_produced(16, PARTIAL_F32, m, m, p, dim3(1, 1, 1), nullptr);
    if (!rc) rc = launch_produced(16, ADD_F32, m, m, p, dim3(1, 1, 1), nullptr);
    g_configure_only = false;
    return rc;
}
