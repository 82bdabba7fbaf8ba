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


// ---- temperature sampling over a large vocabulary, in two stages ------------------------------------
// The one-block-per-row kernel above walks a 65,536-entry row three times with 16 to 64 blocks on the
// whole GPU (114 us measured).  Here SAMPLE_PARTS blocks per row each take a contiguous stretch: its
// greedy pick, its max m_j and s_j = sum exp((v - m_j)/T).  The second stage (a block per row) scales the
// parts to the row's max M (f_j = exp((m_j - M)/T)), walks them in vocabulary order to the part that holds
// target = u * sum_j f_j s_j, and repeats that part's sums to find the entry.  Both stages compute a part's
// sums by the same function (a thread owns a contiguous chunk, chunks are scanned in thread order), so the
// second stage meets exactly the numbers the first one added up.
constexpr int SAMPLE_PARTS = 32;
constexpr int SAMPLE_PART_THREADS = 256;

struct PartSum { float incl, excl, total; };

// Inclusive / exclusive prefix of one value per thread in thread order, and the block's total.
__device__ __forceinline__ PartSum block_scan(float own, float* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        float t = lane < nw ? scratch[lane] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += up;
        }
        scratch[lane] = t;                       // inclusive over warps
        if (lane == 31) scratch[32] = t;
    }
    __syncthreads();
    const float before = warp > 0 ? scratch[warp - 1] : 0.f;
    PartSum r;
    r.incl = before + incl;
    r.excl = r.incl - own;
    r.total = scratch[((blockDim.x + 31) >> 5) - 1];
    return r;
}

// The stretch of part j and the chunk of this thread inside it.
__device__ __forceinline__ void part_chunk(int vocab, int part, int& lo, int& hi, int& clo, int& chi) {
    const int per = (vocab + SAMPLE_PARTS - 1) / SAMPLE_PARTS;
    lo = min(vocab, part * per);
    hi = min(vocab, lo + per);
    const int chunk = (per + SAMPLE_PART_THREADS - 1) / SAMPLE_PART_THREADS;
    clo = min(hi, lo + (int)threadIdx.x * chunk);
    chi = min(hi, clo + chunk);
}

__device__ __forceinline__ float chunk_exp_sum(const float* __restrict__ row, int clo, int chi, float m, float invT) {
    float s = 0.f;
    for (int i = clo; i < chi; ++i) {
        const float v = row[i];
        if (v == v) s += expf((v - m) * invT);
    }
    return s;
}

__global__ void __launch_bounds__(SAMPLE_PART_THREADS)
sample_partial_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                      float* __restrict__ part_max, float* __restrict__ part_sum, int* __restrict__ part_idx,
                      int vocab, int ld) {
    __shared__ MaxIdx mscratch[33];
    __shared__ float fscratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, part = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    int lo, hi, clo, chi;
    part_chunk(vocab, part, lo, hi, clo, chi);
    MaxIdx m{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > m.v || (v == m.v && i < m.i)) { m.v = v; m.i = i; }
    }
    m = block_argmax(m, mscratch);
    const float T = temperature[r];
    float total = 0.f;
    if (T > 0.f && m.i != 0x7fffffff && m.v > -INFINITY)          // block-uniform: every thread holds the same m
        total = block_scan(chunk_exp_sum(row, clo, chi, m.v, 1.0f / T), fscratch).total;
    if (threadIdx.x == 0) {
        part_max[r * SAMPLE_PARTS + part] = m.v;
        part_idx[r * SAMPLE_PARTS + part] = m.i;
        part_sum[r * SAMPLE_PARTS + part] = total;
    }
}

__global__ void __launch_bounds__(SAMPLE_PART_THREADS)
sample_final_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                    const float* __restrict__ uniform, const float* __restrict__ part_max,
                    const float* __restrict__ part_sum, const int* __restrict__ part_idx,
                    int* __restrict__ out, int vocab, int ld) {
    __shared__ float fscratch[33];
    __shared__ float s_run, s_f, s_target, s_m;
    __shared__ int s_owner, s_best, s_first;
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature[r];
    if (threadIdx.x == 0) {
        // the row's greedy pick (larger value, then smaller index) and max
        MaxIdx best{-INFINITY, 0x7fffffff};
        for (int j = 0; j < SAMPLE_PARTS; ++j)
            best = better(best, MaxIdx{part_max[r * SAMPLE_PARTS + j], part_idx[r * SAMPLE_PARTS + j]});
        s_best = best.i;
        s_owner = -1;
        s_first = 0x7fffffff;
        if (T > 0.f && best.i != 0x7fffffff) {
            const float invT = 1.0f / T;
            float f[SAMPLE_PARTS], total = 0.f;
            for (int j = 0; j < SAMPLE_PARTS; ++j) {
                const float sj = part_sum[r * SAMPLE_PARTS + j];
                f[j] = sj > 0.f ? expf((part_max[r * SAMPLE_PARTS + j] - best.v) * invT) : 0.f;
                total += f[j] * sj;
            }
            const float target = uniform[r] * total;
            // the first part whose sum carries the running sum past the target; if rounding leaves the target
            // beyond every sum, the last part with any weight
            float run = 0.f, before_owner = 0.f;
            int owner = -1;
            for (int j = 0; j < SAMPLE_PARTS; ++j) {
                const float pj = f[j] * part_sum[r * SAMPLE_PARTS + j];
                if (pj > 0.f) {
                    owner = j;
                    before_owner = run;
                    if (run + pj > target) break;
                }
                run += pj;
            }
            run = before_owner;
            s_owner = owner;
            s_run = run;
            s_f = owner >= 0 ? f[owner] : 0.f;
            s_target = target;
            s_m = owner >= 0 ? part_max[r * SAMPLE_PARTS + owner] : 0.f;
        }
    }
    __syncthreads();
    const int owner = s_owner;
    if (owner < 0) {                                              // greedy row, or nothing to sample from
        if (threadIdx.x == 0) out[r] = s_best == 0x7fffffff ? 0 : s_best;
        return;
    }
    const float run = s_run, f = s_f, target = s_target, m = s_m, invT = 1.0f / T;
    int lo, hi, clo, chi;
    part_chunk(vocab, owner, lo, hi, clo, chi);
    const float own = chunk_exp_sum(row, clo, chi, m, invT);
    const PartSum ps = block_scan(own, fscratch);
    if (own > 0.f && run + f * ps.incl > target) atomicMin(&s_first, (int)threadIdx.x);
    __syncthreads();
    if ((int)threadIdx.x == s_first) {
        float acc = ps.incl - own;
        int chosen = -1, last = -1;
        for (int i = clo; i < chi; ++i) {
            const float v = row[i];
            if (v == v) {
                acc += expf((v - m) * invT);
                last = i;
                if (run + f * acc > target) { chosen = i; break; }
            }
        }
        out[r] = chosen >= 0 ? chosen : last;
    }
    if (s_first == 0x7fffffff && threadIdx.x == 0) out[r] = s_best;   // rounding left the target beyond the last sum
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

// Temperature (and greedy) rows over a large vocabulary in two stages.  part_f: 2 * n_rows * 32 floats,
// part_idx: n_rows * 32 ints of scratch.
extern "C" int imparo_sample_rows_parts(const float* logits, const float* temperature, const float* uniform, int* out,
                                        float* part_f, int* part_idx, int n_rows, int vocab, int ld, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!temperature || !uniform) return -7;
    if (n_rows > 65535) return -2;
    float* part_max = part_f;
    float* part_sum = part_f + (size_t)n_rows * imparo::SAMPLE_PARTS;
    launch(imparo::sample_partial_kernel, dim3(imparo::SAMPLE_PARTS, n_rows), dim3(imparo::SAMPLE_PART_THREADS), 0, stream,
           logits, temperature, part_max, part_sum, part_idx, vocab, ld);
    launch(imparo::sample_final_kernel, dim3(n_rows), dim3(imparo::SAMPLE_PART_THREADS), 0, stream, logits, temperature,
           uniform, (const float*)part_max, (const float*)part_sum, (const int*)part_idx, out, vocab, ld);
    IMPARO_CHECK_LAUNCH();
    return 0;
}
