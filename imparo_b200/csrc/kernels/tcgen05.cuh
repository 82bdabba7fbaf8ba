// Pieces shared by the kernels that drive the 5th-generation tensor cores: mbarriers with
// bounded waits, TMA tile loads, shared-memory and instruction descriptors for tcgen05.mma,
// tensor-memory loads, and the host's cache of tensor maps.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>

namespace imparo {
namespace tc {

constexpr int BK = 64;             // bfloat16 elements per 128-byte row of a tile: one swizzle atom wide
constexpr int UMMA_K = 16;
constexpr uint32_t WAIT_LIMIT = 4000000u;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one look: has the phase of this parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// false when the wait ran out (after `limit` polls)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = WAIT_LIMIT) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// A tile of shared memory ([z][y][x], dense) written to a 3-D tensor by the TMA engine.  Elements outside the
// tensor are not written (tiles that hang over the last row or column need no masks).  The calling thread must
// wait with tma_store_wait_read() before the shared memory is reused or the CTA exits; the writes themselves are
// complete, like any other of the kernel's, when the grid is.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle: 8-row groups
// are 1024 bytes apart (SBO); the leading-dimension offset is unused for this layout.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                    // LBO (ignored for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // SBO
    d |= (uint64_t)1 << 46;                    // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}
// kind::f16, A and B bfloat16 K-major, D float32
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// CH chunks of 16 accumulator columns with one wait: the loads are issued back to back, and the
// empty statements after the wait keep every use of the values behind it.
template <int CH>
__device__ __forceinline__ void tmem_ld_chunks(uint32_t taddr, float (&v)[CH][16]) {
    uint32_t r[CH][16];
#pragma unroll
    for (int u = 0; u < CH; ++u)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=r"(r[u][0]), "=r"(r[u][1]), "=r"(r[u][2]), "=r"(r[u][3]), "=r"(r[u][4]), "=r"(r[u][5]), "=r"(r[u][6]),
                       "=r"(r[u][7]), "=r"(r[u][8]), "=r"(r[u][9]), "=r"(r[u][10]), "=r"(r[u][11]), "=r"(r[u][12]),
                       "=r"(r[u][13]), "=r"(r[u][14]), "=r"(r[u][15])
                     : "r"(taddr + 16 * u));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int u = 0; u < CH; ++u) {
        asm volatile("" : "+r"(r[u][0]), "+r"(r[u][1]), "+r"(r[u][2]), "+r"(r[u][3]), "+r"(r[u][4]), "+r"(r[u][5]), "+r"(r[u][6]),
                          "+r"(r[u][7]), "+r"(r[u][8]), "+r"(r[u][9]), "+r"(r[u][10]), "+r"(r[u][11]), "+r"(r[u][12]),
                          "+r"(r[u][13]), "+r"(r[u][14]), "+r"(r[u][15]) :: "memory");
#pragma unroll
        for (int i = 0; i < 16; ++i) v[u][i] = __uint_as_float(r[u][i]);
    }
}


// ---- host: tensor maps ------------------------------------------------------------------------
// A [rows, cols] bfloat16 matrix with row stride ld (elements), tiles of box_rows x 64 elements,
// 128-byte swizzle.  Maps are cached per translation unit by (pointer, extents, box).
static PFN_cuTensorMapEncodeTiled g_encode = nullptr;
static std::mutex g_mutex;
struct MapKey {
    const void* ptr; uint64_t rows, cols, ld; uint32_t box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (k.rows * 1315423911u) ^ (k.cols << 20) ^ (k.ld << 7) ^ k.box_rows;
    }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

static inline int get_map(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) return -20;
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    }
    const MapKey key{ptr, rows, cols, ld, box_rows};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    if (g_maps.size() > 4096) g_maps.clear();
    CUtensorMap m;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -21;
    g_maps.emplace(key, m);
    *out = m;
    return 0;
}

// A 3-D map over split partials [splits][T][N] in 32-bit, no swizzle, for stores of boxes [1][box_t][128] (x = the
// row of W, the innermost dimension).  N must be a multiple of 4 (16-byte rows) and ptr 16-byte aligned.
static inline int get_map_partials(const void* ptr, uint64_t N, uint64_t T, uint64_t splits, uint32_t box_t, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) return -20;
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    }
    const MapKey key{ptr, T, N, splits, box_t | 0x80000000u};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    if (g_maps.size() > 4096) g_maps.clear();
    CUtensorMap m;
    const cuuint64_t dims[3] = {N, T, splits};
    const cuuint64_t strides[2] = {N * 4, T * N * 4};
    const cuuint32_t box[3] = {128, box_t, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -21;
    g_maps.emplace(key, m);
    *out = m;
    return 0;
}

}  // namespace tc
}  // namespace imparo
