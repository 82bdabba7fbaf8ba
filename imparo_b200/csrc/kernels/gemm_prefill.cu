// bfloat16 matrix product for prompt-sized batches on the 5th-generation tensor cores:
//     out[T, N] (+)= X[T, K] * W[N, K]^T        (both operands K-major, 32-bit accumulation)
//
// Where gemm_tcgen05.cu streams weights for a handful of tokens, this kernel is bound by the
// tensor cores: hundreds to thousands of tokens, every weight tile reused by many token tiles.
//   * The tokens are the MMA's M operand (128 per tile, tensor-memory lanes = tokens), the rows
//     of W its N operand (256 per tile): one tcgen05.mma is 128 x 256 x 16.
//   * Persistent CTAs, one per SM, walk the output tiles in an order that keeps CTAs that run
//     together on the same rows of W (W is read from HBM once, X stays in the L2).
//   * Warp 0 feeds a 4-stage ring of (X tile 16 KB | W tile 32 KB) by TMA (128-byte swizzle, no
//     multicast); warp 1 issues the MMAs; the accumulator lives in tensor memory, twice: while
//     warps 2-5 read one accumulator out (tcgen05.ld) and run the epilogue, the MMAs of the next
//     tile already fill the other.
//   * Epilogues, all on the accumulator in registers, a token row per thread:
//       store bfloat16 | store float32 | add into float32 (the residual stream) |
//       SwiGLU: the tile's 256 rows of W are 128 gate rows and the 128 up rows of the same
//       features, h = silu(gate) * up is written as bfloat16 [T, F]
//       (imparo-cpu/src/ops.rs:73-78; imparo-model/src/lfm2/workflow_cpu.rs:307-313): the
//       [T, 2F] intermediate and the activation kernel's pass over it disappear.
// The reference hands these products to cuBLAS (imparo-cuda/native/bf16_bounded_gemm.cuh:4-28).
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records
// IMPARO_ST_WAIT_LIMIT in the status word, stops waiting, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace imparo {
namespace tcp {

using namespace imparo::tc;

constexpr int TM = 128;            // tokens per tile (MMA M)
constexpr int TN = 256;            // rows of W per tile (MMA N); SwiGLU: 128 gate + 128 up
constexpr int STAGES = 4;
constexpr int THREADS = 192;       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr uint32_t A_BYTES = TM * BK * 2, B_BYTES = TN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t TMEM_COLS = 2 * TN;
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + 256;

enum Epilogue { STORE_BF16 = 0, STORE_F32 = 1, ADD_F32 = 2, SWIGLU_BF16 = 3 };

struct Params {
    void* out;               // [T, ldo]
    int* status;
    int T, N, K, ldo;        // N = output columns (SwiGLU: F, W has 2F rows)
    int kblocks;             // ceil(K / BK)
    int m_tiles, n_tiles;
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// keeps every use of the loaded registers behind the wait
__device__ __forceinline__ void pin32(uint32_t (&r)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) asm volatile("" : "+r"(r[i]) :: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// tile index -> (token tile, row tile): consecutive indices share a row tile of W
__device__ __forceinline__ void tile_of(int idx, const Params& p, int& tm, int& tn) {
    tn = idx / p.m_tiles;
    tm = idx - tn * p.m_tiles;
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_prefill_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* aux = smem + STAGES * STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(aux);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;           // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles_total = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
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
            // W is written by no kernel: the first ring of W tiles is requested before the wait on
            // the previous kernel.  g counts k-blocks over all of this CTA's tiles.
            auto load_w = [&](int g, int tn, int kb) {
                const int s = g % STAGES;
                uint8_t* b = smem + s * STAGE_BYTES + A_BYTES;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                if (EPI == SWIGLU_BF16) {
                    tma_load_2d(b, &map_w, &full[s], kb * BK, tn * 128);                      // 128 gate rows
                    tma_load_2d(b + B_BYTES / 2, &map_w, &full[s], kb * BK, p.N + tn * 128);  // their 128 up rows
                } else {
                    tma_load_2d(b, &map_w, &full[s], kb * BK, tn * TN);
                }
            };
            auto load_x = [&](int g, int tm, int kb) {
                const int s = g % STAGES;
                tma_load_2d(smem + s * STAGE_BYTES, &map_x, &full[s], kb * BK, tm * TM);
            };
            pdl_trigger();
            int g = 0;
            bool ok = true, first = true;
            for (int idx = blockIdx.x; idx < n_tiles_total && ok; idx += gridDim.x) {
                int tm, tn;
                tile_of(idx, p, tm, tn);
                int kb = 0;
                if (first) {
                    const int early = p.kblocks < STAGES ? p.kblocks : STAGES;
                    for (int i = 0; i < early; ++i) load_w(i, tn, i);
                    pdl_wait();
                    for (int i = 0; i < early; ++i) load_x(i, tm, i);
                    g = kb = early;
                    first = false;
                }
                for (; kb < p.kblocks; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (g >= STAGES && !mbar_wait(&empty[s], ((g / STAGES) - 1) & 1)) {
                        report(p.status, IMPARO_ST_WAIT_LIMIT, 20, idx, kb);
                        ok = false;
                        break;
                    }
                    load_w(g, tn, kb);
                    load_x(g, tm, kb);
                }
            }
            if (first) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(TM, TN);
            const uint64_t desc_a0 = smem_desc(smem_u32(smem)), desc_b0 = smem_desc(smem_u32(smem) + A_BYTES);
            int g = 0, it = 0;
            bool ok = true;
            for (int idx = blockIdx.x; idx < n_tiles_total && ok; idx += gridDim.x, ++it) {
                const int b = it & 1, use = it >> 1;
                if (use > 0 && !mbar_wait(&acc_empty[b], (use - 1) & 1)) {       // the epilogue has read this accumulator out
                    report(p.status, IMPARO_ST_WAIT_LIMIT, 21, idx, b);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)b * TN;
                for (int kb = 0; kb < p.kblocks; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (!mbar_wait(&full[s], (g / STAGES) & 1)) {
                        report(p.status, IMPARO_ST_WAIT_LIMIT, 22, idx, kb);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // the stage's two descriptors are the ring's first ones plus the stage's offset / 16 (the address
                    // field is the low 14 bits and never carries), a slice of 16 along K is 32 bytes further: the
                    // issuing thread spends its cycles on the products, not on their operands' descriptors
                    const uint64_t da = desc_a0 + (uint64_t)((s * STAGE_BYTES) >> 4), db = desc_b0 + (uint64_t)((s * STAGE_BYTES) >> 4);
                    umma(d_tmem, da, db, idesc, kb > 0 ? 1u : 0u);
#pragma unroll
                    for (int k = 1; k < BK / UMMA_K; ++k)
                        umma(d_tmem, da + (uint64_t)((k * UMMA_K * 2) >> 4), db + (uint64_t)((k * UMMA_K * 2) >> 4), idesc, 1u);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +32; a lane is a token ----
        const int quad = warp & 3;
        pdl_wait();                                             // before any global write or residual read
        int it = 0;
        for (int idx = blockIdx.x; idx < n_tiles_total; idx += gridDim.x, ++it) {
            int tm, tn;
            tile_of(idx, p, tm, tn);
            const int b = it & 1, use = it >> 1;
            const bool ok = p.kblocks == 0 || mbar_wait(&acc_full[b], use & 1);
            if (!ok) {
                if (lane == 0) report(p.status, IMPARO_ST_WAIT_LIMIT, 23, idx, b);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)b * TN;
            const int t = tm * TM + quad * 32 + lane;
            const bool live = t < p.T;
            if (EPI == SWIGLU_BF16) {
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)t * p.ldo;
                const int f0 = tn * 128;
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    uint32_t gr[32], ur[32];
                    tmem_ld32(taddr + c, gr);
                    tmem_ld32(taddr + 128 + c, ur);
                    tmem_ld_wait();
                    pin32(gr); pin32(ur);
                    if (c + 32 >= 128) {
                        // everything of this accumulator is in registers: hand it back to the MMAs
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[b])) : "memory");
                    }
                    if (live) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            const int f = f0 + c + j;
                            if (f < p.N) {                      // N is a multiple of 8: whole 16-byte groups
                                uint32_t w[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float g0 = __uint_as_float(gr[j + 2 * e]), g1 = __uint_as_float(gr[j + 2 * e + 1]);
                                    const float u0 = __uint_as_float(ur[j + 2 * e]), u1 = __uint_as_float(ur[j + 2 * e + 1]);
                                    w[e] = pack_bf16(silu_bf16(g0) * u0, silu_bf16(g1) * u1);
                                }
                                *reinterpret_cast<uint4*>(out + f) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            } else {
                const int n0 = tn * TN;
#pragma unroll 1
                for (int c = 0; c < TN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_ld_wait();
                    pin32(r);
                    if (c + 32 >= TN) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[b])) : "memory");
                    }
                    if (!live) continue;
                    if (EPI == STORE_BF16) {
                        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)t * p.ldo;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            const int n = n0 + c + j;
                            if (n < p.N)
                                *reinterpret_cast<uint4*>(out + n) =
                                    make_uint4(pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                                               pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                                               pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                                               pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
                        }
                    } else {
                        float* out = reinterpret_cast<float*>(p.out) + (size_t)t * p.ldo;
                        if (EPI == ADD_F32) {
                            // all reads of the stream before any write (the compiler cannot prove the addresses differ)
                            float4 old[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int n = n0 + c + 4 * j;
                                old[j] = n < p.N ? *reinterpret_cast<const float4*>(out + n) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int n = n0 + c + 4 * j;
                                if (n < p.N)
                                    *reinterpret_cast<float4*>(out + n) =
                                        make_float4(old[j].x + __uint_as_float(r[4 * j]), old[j].y + __uint_as_float(r[4 * j + 1]),
                                                    old[j].z + __uint_as_float(r[4 * j + 2]), old[j].w + __uint_as_float(r[4 * j + 3]));
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int n = n0 + c + 4 * j;
                                if (n < p.N)
                                    *reinterpret_cast<float4*>(out + n) =
                                        make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                    __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                            }
                        }
                    }
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

template <int EPI>
static int launch_prefill(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int ctas, cudaStream_t stream) {
    auto kern = gemm_prefill_kernel<EPI>;
    static bool configured = false;
    cudaError_t e;
    if (!configured) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    e = timeline_note(reinterpret_cast<const void*>(kern));
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = imparo_pdl_enabled() ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kern, mw, mx, p);
    return e == cudaSuccess ? 0 : (int)e;
}

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 1;
    }
    return n;
}

}  // namespace tcp
}  // namespace imparo

using namespace imparo::tcp;

// x: [T, K] bfloat16 with row stride ldx (elements), inside a buffer of x_rows_alloc rows.
// w: [N, K] bfloat16 dense (SwiGLU: [2N, K], gate rows then up rows).  out: [T, ldo].
// epilogue: 0 store bfloat16, 1 store float32, 2 add into float32, 3 SwiGLU (bfloat16 [T, N]).
// Refused (-23): K or ldx not a multiple of 8, operands not 16-byte aligned, N or ldo not a
// multiple of 8 (4 for the float32 outputs), out not 16-byte aligned: the caller then takes the
// library product.
extern "C" int imparo_gemm_prefill(const void* x, int ldx, int x_rows_alloc, const void* w, void* out, int ldo,
                                   int T, int N, int K, int epilogue, int* status, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0) return -23;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return -23;
    const bool f32_out = epilogue == STORE_F32 || epilogue == ADD_F32;
    if (N % (f32_out ? 4 : 8) != 0 || ldo % (f32_out ? 4 : 8) != 0) return -23;
    if (epilogue < 0 || epilogue > 3) return -22;
    const int w_rows = epilogue == SWIGLU_BF16 ? 2 * N : N;
    CUtensorMap mw, mx;
    int rc = get_map(w, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, epilogue == SWIGLU_BF16 ? 128u : (uint32_t)TN, &mw);
    if (rc) return rc;
    rc = get_map(x, (uint64_t)(x_rows_alloc > T ? x_rows_alloc : T), (uint64_t)K, (uint64_t)ldx, (uint32_t)TM, &mx);
    if (rc) return rc;
    Params p = {};
    p.out = out; p.status = status;
    p.T = T; p.N = N; p.K = K; p.ldo = ldo; p.kblocks = (K + BK - 1) / BK;
    p.m_tiles = (T + TM - 1) / TM;
    p.n_tiles = epilogue == SWIGLU_BF16 ? (N + 127) / 128 : (N + TN - 1) / TN;
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles > (1 << 30)) return -2;
    const int ctas = (int)(tiles < sm_count() ? tiles : sm_count());
    switch (epilogue) {
        case STORE_BF16: return launch_prefill<STORE_BF16>(mw, mx, p, ctas, stream);
        case STORE_F32: return launch_prefill<STORE_F32>(mw, mx, p, ctas, stream);
        case ADD_F32: return launch_prefill<ADD_F32>(mw, mx, p, ctas, stream);
        default: return launch_prefill<SWIGLU_BF16>(mw, mx, p, ctas, stream);
    }
}
