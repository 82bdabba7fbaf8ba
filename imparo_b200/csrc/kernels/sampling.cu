// Sampling over rows of 32-bit logits.
//
// Greedy follows the reference's rule: the smallest index that attains the maximum, NaN
// never wins, an all-NaN row gives 0 (imparo-cpu/src/ops.rs:628-640;
// imparo-cuda/native/imparo_cuda.cu:5531-5562 k_argmax_rows).  The reference has no
// temperature sampling (imparo-server/src/main.rs:3383-3390 ignores its temperature);
// here p = softmax(logits / T) in 32-bit and the pick is the first index whose running
// sum of p, taken in vocabulary order, exceeds u * total, with u in [0,1) given per row.
#include "common.cuh"

namespace imparo {

constexpr int SAMPLE_THREADS = 1024;

struct MaxIdx { float v; int i; };

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    // larger value wins; on equal values the smaller index wins
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ MaxIdx block_argmax(MaxIdx m, MaxIdx* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, m.v, o), __shfl_xor_sync(0xffffffffu, m.i, o)};
        m = better(m, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        MaxIdx t = lane < nw ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// One block per row.  temperature[r] <= 0 means greedy.  Each thread owns one contiguous
// stretch of the vocabulary, so the running sum is taken in vocabulary order.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, int* __restrict__ out, int vocab, int ld) {
    __shared__ MaxIdx mscratch[33];
    __shared__ float fscratch[33];
    __shared__ float part[SAMPLE_THREADS];
    __shared__ int pick;
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = min(vocab, (int)threadIdx.x * per), hi = min(vocab, lo + per);

    MaxIdx m{-INFINITY, 0x7fffffff};
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v > m.v) { m.v = v; m.i = i; }      // NaN compares false: never wins
    }
    m = block_argmax(m, mscratch);
    const float T = temperature ? temperature[r] : 0.f;
    if (!(T > 0.f) || m.i == 0x7fffffff) {
        if (threadIdx.x == 0) out[r] = m.i == 0x7fffffff ? 0 : m.i;
        return;
    }
    const float invT = 1.0f / T;
    float s = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += expf((v - m.v) * invT);
    }
    part[threadIdx.x] = s;
    const float total = block_sum(s, fscratch);
    const float target = uniform[r] * total;
    if (threadIdx.x == 0) pick = -1;
    __syncthreads();
    // serial prefix over the per-thread sums by one thread: 1024 adds, in order
    if (threadIdx.x == 0) {
        float run = 0.f;
        int owner = blockDim.x - 1;
        for (int k = 0; k + 1 < (int)blockDim.x; ++k) {
            if (run + part[k] > target) { owner = k; break; }
            run += part[k];
        }
        fscratch[0] = run;
        pick = owner;
    }
    __syncthreads();
    if ((int)threadIdx.x == pick) {
        float run = fscratch[0];
        int chosen = -1;
        for (int i = lo; i < hi; ++i) {
            const float v = row[i];
            if (v == v) {
                run += expf((v - m.v) * invT);
                if (run > target) { chosen = i; break; }
            }
        }
        if (chosen < 0) chosen = m.i;     // rounding left the target beyond the last sum
        out[r] = chosen;
    }
}

// Greedy only, for many rows or a large vocabulary: ARGMAX_PARTS blocks per row each find
// the best of a contiguous stretch, then one warp per row folds them (same rule: larger
// value, then smaller index).
constexpr int ARGMAX_PARTS = 32;

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ part_val, int* __restrict__ part_idx,
                      int vocab, int ld) {
    __shared__ MaxIdx scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, part = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int per = (vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
    const int lo = min(vocab, part * per), hi = min(vocab, lo + per);
    MaxIdx m{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > m.v || (v == m.v && i < m.i)) { m.v = v; m.i = i; }
    }
    m = block_argmax(m, scratch);
    if (threadIdx.x == 0) { part_val[r * ARGMAX_PARTS + part] = m.v; part_idx[r * ARGMAX_PARTS + part] = m.i; }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, lane = threadIdx.x;
    MaxIdx m{part_val[r * ARGMAX_PARTS + lane], part_idx[r * ARGMAX_PARTS + lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, m.v, o), __shfl_xor_sync(0xffffffffu, m.i, o)};
        m = better(m, other);
    }
    if (lane == 0) out[r] = m.i == 0x7fffffff ? 0 : m.i;
}

}  // namespace imparo

// part_val / part_idx: scratch of n_rows * 32 entries each.
// token_ids[i] = prev[src[i]] where src[i] >= 0: a step takes the ids the step before it sampled
// straight from that step's output on the device (rows with src < 0 keep the id the host wrote)
namespace imparo {
__global__ void take_sampled_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ src,
                                           const int* __restrict__ prev, int n, int n_prev) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int s = src[i];
        if (s >= 0 && s < n_prev) token_ids[i] = prev[s];
    }
}
}  // namespace imparo

extern "C" int imparo_take_sampled_tokens(int* token_ids, const int* src, const int* prev, int n, int n_prev,
                                          cudaStream_t stream) {
    if (n <= 0) return 0;
    launch(imparo::take_sampled_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, token_ids, src, prev, n, n_prev);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_argmax_rows(const float* logits, int* out, float* part_val, int* part_idx,
                                  int n_rows, int vocab, int ld, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > 65535) return -2;
    dim3 grid(imparo::ARGMAX_PARTS, n_rows);
    launch(imparo::argmax_partial_kernel, grid, dim3(256), 0, stream, logits, part_val, part_idx, vocab, ld);
    launch(imparo::argmax_final_kernel, dim3(n_rows), dim3(32), 0, stream, part_val, part_idx, out);
    IMPARO_CHECK_LAUNCH();
    return 0;
}

extern "C" int imparo_sample_rows(const float* logits, const float* temperature, const float* uniform, int* out,
                                  int n_rows, int vocab, int ld, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (temperature && !uniform) return -7;
    launch(imparo::sample_rows_kernel, dim3(n_rows), dim3(imparo::SAMPLE_THREADS), 0, stream, logits, temperature, uniform, out, vocab, ld);
    IMPARO_CHECK_LAUNCH();
    return 0;
}
