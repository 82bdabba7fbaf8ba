// Gated causal depthwise convolution with per-request rolling state, for a ragged batch.
//
// Formula (zeraix/imparo, imparo-cpu/src/ops.rs:109-167; imparo-cuda/native/lfm2_ops.cuh:48-97):
//   rows of bcx are [b | c | x];  v[t] = b[t]*x[t];  seq = state ++ v  (state = the taps-1
//   raw v before this portion, oldest first, zeros for a fresh request);
//   sum[t] = sum_k w[ch,k] * seq[t+k]  (tap 0 meets the oldest value);  y[t] = c[t]*sum[t];
//   state' = the last taps-1 values of seq (partly the old state when the portion is
//   shorter than taps-1).  A bias, which the reference does not have, is added to sum
//   before the gate.
//
// One launch does output and state.  A thread owns (token, channel) — or, for prompt portions in
// bfloat16, (token, eight channels).  Tokens at least taps-1 into their portion need only bcx.
// The thread of a portion's FIRST token also computes the outputs of the next taps-2 tokens and
// then writes the new state; it reads the whole old state into registers first, and no other
// thread touches that state, so the update in place is race-free.  The input may also be the
// split partials of the product before (summed here), see ConvIn.
#include "common.cuh"

namespace imparo {

constexpr int MAX_TAPS = 16;

// The input rows [b | c | x]: a stored tensor of T, or the partial results of a product that was
// cut along K (float [parts][tokens][3 * width]).  Partials are summed in split order and rounded
// to T, which is what the product's own fold would have stored.
// MODE 0: a tensor; 1: at most four partials (straight-line code, so that the loads of the
// several values a thread needs are all in flight together); 2: any number of partials.
template <typename T, int MODE>
struct ConvIn {
    const T* rows;
    const float* part;
    int parts;
    size_t part_stride;
    __device__ __forceinline__ float at(size_t idx) const {
        if (MODE == 0) return to_f32(rows[idx]);
        float acc = 0.f;
        if (MODE == 1) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = u < parts ? __ldcg(part + (size_t)u * part_stride + idx) : 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) if (u < parts) acc += v[u];
        } else {
            for (int s0 = 0; s0 < parts; s0 += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = s0 + u < parts ? __ldcg(part + (size_t)(s0 + u) * part_stride + idx) : 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u) if (s0 + u < parts) acc += v[u];
            }
        }
        return to_f32(from_f32<T>(acc));
    }
};

// The thread of a portion's first token, for one channel: outputs of the first min(n, taps-1)
// tokens from the old state, then the new state.  wk: this channel's taps (loaded by the caller,
// before it waited for the previous kernel).  Everything the outputs need is requested in one
// batch of loads: a decode token costs one round trip to memory after the wait.
template <typename T, int MODE>
__device__ __forceinline__ void conv_portion_head(const ConvIn<T, MODE>& bcx, const float* wk, float b0,
                                                  float* __restrict__ state, int slot,
                                                  T* __restrict__ y, int item, int start, int n, int ch,
                                                  int width, int taps, int n_slots, int* status) {
    const int hist = taps - 1;
    const size_t stride = (size_t)3 * width;
    if (slot < 0 || slot >= n_slots) {
        if (ch == 0) report(status, IMPARO_ST_SLOT_RANGE, 4, item, slot);
        return;
    }
    float* st = state + (size_t)slot * hist * width + ch;
    // seq[e], e in [0, hist + m): the old state then the first m values of this portion
    float seq[2 * MAX_TAPS], gate[MAX_TAPS];
    const int m = min(n, hist);
#pragma unroll
    for (int e = 0; e < MAX_TAPS; ++e) if (e < hist) seq[e] = st[(size_t)e * width];
#pragma unroll
    for (int e = 0; e < MAX_TAPS; ++e) {
        if (e < m) {
            const size_t r = (size_t)(start + e) * stride;
            seq[hist + e] = bcx.at(r + ch) * bcx.at(r + 2 * (size_t)width + ch);
            gate[e] = bcx.at(r + width + ch);
        }
    }
    for (int e = 0; e < m; ++e) {
        float acc = 0.f;
        for (int k = 0; k < taps; ++k) acc += wk[k] * seq[e + k];
        acc += b0;
        y[(size_t)(start + e) * width + ch] = from_f32<T>(gate[e] * acc);
    }
    // new state slot s = seq_full[n + s]
    for (int s = 0; s < hist; ++s) {
        const int e = n + s;
        float v;
        if (e < hist + m) {
            v = seq[e];
        } else {
            const size_t r = (size_t)(start + e - hist) * stride;
            v = bcx.at(r + ch) * bcx.at(r + 2 * (size_t)width + ch);
        }
        st[(size_t)s * width] = v;
    }
}

// The batch description (which request a token belongs to, where its portion starts, its state
// slot) comes from the host before the step and the taps are weights: both are read before the
// wait on the previous kernel, so that after it only activations and state remain to be fetched.
template <typename T, int MODE>
__global__ void gated_conv_kernel(const ConvIn<T, MODE> bcx, const float* __restrict__ w,
                                  const float* __restrict__ bias, float* __restrict__ state,
                                  const int* __restrict__ item_row_start, const int* __restrict__ item_of_token,
                                  const int* __restrict__ item_slot, T* __restrict__ y,
                                  int n_tok, int width, int taps, int n_slots, int* status) {
    pdl_trigger();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_tok * width) return;
    const int t = (int)(idx / width), ch = (int)(idx % width);
    const int item = item_of_token[t];
    const int start = item_row_start[item];
    const int n = item_row_start[item + 1] - start;
    const int rel = t - start;
    const int hist = taps - 1;
    if (rel > 0 && rel < hist) return;           // written by the thread of the portion's first token
    const int slot = rel == 0 ? item_slot[item] : 0;
    const size_t stride = (size_t)3 * width;
    float wk[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) wk[k] = k < taps ? w[(size_t)ch * taps + k] : 0.f;
    const float b0 = bias ? bias[ch] : 0.f;
    pdl_wait();

    if (rel >= hist) {
        float v[MAX_TAPS];
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k) {
            if (k < taps) {
                const size_t r = (size_t)(t - hist + k) * stride;
                v[k] = bcx.at(r + ch) * bcx.at(r + 2 * (size_t)width + ch);
            }
        }
        const float gate = bcx.at((size_t)t * stride + width + ch);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k) if (k < taps) acc += wk[k] * v[k];
        acc += b0;
        y[(size_t)t * width + ch] = from_f32<T>(gate * acc);
        return;
    }
    if (n == 1 && slot >= 0 && slot < n_slots) {
        // a decode token: everything in registers, one batch of loads
        float* st = state + (size_t)slot * hist * width + ch;
        float sv[MAX_TAPS];
#pragma unroll
        for (int e = 0; e < MAX_TAPS - 1; ++e) sv[e] = e < hist ? st[(size_t)e * width] : 0.f;
        const size_t r = (size_t)t * stride;
        const float bx = bcx.at(r + ch) * bcx.at(r + 2 * (size_t)width + ch);
        const float gate = bcx.at(r + width + ch);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k) {
            if (k < hist) acc += wk[k] * sv[k];
            else if (k == hist) acc += wk[k] * bx;
        }
        acc += b0;
        y[(size_t)t * width + ch] = from_f32<T>(gate * acc);
#pragma unroll
        for (int e = 0; e < MAX_TAPS - 1; ++e)
            if (e < hist) st[(size_t)e * width] = (e + 1 < hist) ? sv[e + 1] : bx;
        return;
    }
    conv_portion_head<T, MODE>(bcx, wk, b0, state, slot, y, item, start, n, ch, width, taps, n_slots, status);
}

// bfloat16 with a width that is a multiple of 8, for prompt-sized batches: a thread owns eight
// consecutive channels of one token and moves 16 bytes at a time.  Same sums in the same order
// as gated_conv_kernel; the thread of a portion's first token walks its eight channels through
// conv_portion_head.  TAPS > 0: the number of taps is fixed at compile time; the thread's 8 * TAPS
// tap weights are contiguous and come as 16-byte loads, and the loads of all taps' rows are in
// flight together.  TAPS == 0: any number of taps.
template <int TAPS>
__global__ void gated_conv_bf16x8_kernel(const __nv_bfloat16* __restrict__ bcx, const float* __restrict__ w,
                                         const float* __restrict__ bias, float* __restrict__ state,
                                         const int* __restrict__ item_row_start, const int* __restrict__ item_of_token,
                                         const int* __restrict__ item_slot, __nv_bfloat16* __restrict__ y,
                                         int n_tok, int width, int taps_rt, int n_slots, int* status) {
    pdl_trigger();
    const int taps = TAPS > 0 ? TAPS : taps_rt;
    const int per_row = width >> 3;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_tok * per_row) return;
    const int t = (int)(idx / per_row), ch = (int)(idx % per_row) << 3;
    const int hist = taps - 1;
    const int item = item_of_token[t];
    const int start = item_row_start[item];
    const int rel = t - start;
    // the thread's tap weights: w[(ch + i) * taps + k], 8 * taps consecutive floats
    constexpr int NW = TAPS > 0 ? 8 * TAPS : 1;
    float wv[NW];
    if (TAPS > 0) {
        const float4* wp = reinterpret_cast<const float4*>(w + (size_t)ch * TAPS);
#pragma unroll
        for (int q4 = 0; q4 < 2 * TAPS; ++q4) {
            const float4 f = __ldg(wp + q4);
            wv[4 * q4] = f.x; wv[4 * q4 + 1] = f.y; wv[4 * q4 + 2] = f.z; wv[4 * q4 + 3] = f.w;
        }
    }
    pdl_wait();
    if (rel < hist) {
        if (rel != 0) return;
        const int n = item_row_start[item + 1] - start;
        const int slot = item_slot[item];
        for (int i = 0; i < 8; ++i) {
            float wk[MAX_TAPS];
            for (int k = 0; k < taps; ++k) wk[k] = w[(size_t)(ch + i) * taps + k];
            conv_portion_head<__nv_bfloat16, 0>(ConvIn<__nv_bfloat16, 0>{bcx, nullptr, 0, 0}, wk, bias ? bias[ch + i] : 0.f, state, slot, y, item, start, n,
                                             ch + i, width, taps, n_slots, status);
        }
        return;
    }
    const size_t stride = (size_t)3 * width;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const uint4 c = *reinterpret_cast<const uint4*>(bcx + (size_t)t * stride + width + ch);
    if (TAPS > 0) {
        uint4 bq[TAPS > 0 ? TAPS : 1], xq[TAPS > 0 ? TAPS : 1];
#pragma unroll
        for (int k = 0; k < TAPS; ++k) {
            const __nv_bfloat16* r = bcx + (size_t)(t - hist + k) * stride;
            bq[k] = *reinterpret_cast<const uint4*>(r + ch);
            xq[k] = *reinterpret_cast<const uint4*>(r + 2 * (size_t)width + ch);
        }
#pragma unroll
        for (int k = 0; k < TAPS; ++k) {
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bq[k]);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xq[k]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 bf = __bfloat1622float2(bp[i]), xf = __bfloat1622float2(xp[i]);
                acc[2 * i] += wv[(2 * i) * TAPS + k] * (bf.x * xf.x);
                acc[2 * i + 1] += wv[(2 * i + 1) * TAPS + k] * (bf.y * xf.y);
            }
        }
    } else {
        for (int k = 0; k < taps; ++k) {
            const __nv_bfloat16* r = bcx + (size_t)(t - hist + k) * stride;
            const uint4 b = *reinterpret_cast<const uint4*>(r + ch);
            const uint4 x = *reinterpret_cast<const uint4*>(r + 2 * (size_t)width + ch);
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 bf = __bfloat1622float2(bp[i]), xf = __bfloat1622float2(xp[i]);
                acc[2 * i] += w[(size_t)(ch + 2 * i) * taps + k] * (bf.x * xf.x);
                acc[2 * i + 1] += w[(size_t)(ch + 2 * i + 1) * taps + k] * (bf.y * xf.y);
            }
        }
    }
    if (bias) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += bias[ch + i];
    }
    const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&c);
    uint4 out;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 cf = __bfloat1622float2(cp[i]);
        op[i] = __floats2bfloat162_rn(cf.x * acc[2 * i], cf.y * acc[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(y + (size_t)t * width + ch) = out;
}

}  // namespace imparo

using namespace imparo;

// bcx: [n_tok, 3 * width] of the dtype; or, when parts > 0, float partial results
// [parts][n_tok][3 * width] (split s at bcx + s * part_stride floats) of a product cut along K,
// which this kernel sums (the dtype then names the output and the rounding of the sum).
extern "C" int imparo_gated_conv(const void* bcx, int dtype, const float* w, const float* bias, float* state,
                                 const int* item_row_start, const int* item_of_token, const int* item_slot,
                                 void* y, int n_tok, int width, int taps, int n_slots, int parts, long long part_stride,
                                 int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (taps < 2 || taps > MAX_TAPS) return -6;
    if (parts < 0 || (parts > 0 && part_stride < (long long)n_tok * 3 * width)) return -2;
    const size_t n = (size_t)n_tok * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    const float* part = parts > 0 ? (const float*)bcx : nullptr;
    const int mode = parts == 0 ? 0 : (parts <= 4 ? 1 : 2);
#define IMPARO_CONV(T_, M_) do { \
        ConvIn<T_, M_> in{(const T_*)bcx, part, parts, (size_t)part_stride}; \
        launch(gated_conv_kernel<T_, M_>, dim3(blocks), dim3(threads), 0, stream, in, w, bias, state, item_row_start, \
               item_of_token, item_slot, (T_*)y, n_tok, width, taps, n_slots, status); } while (0)
    if (dtype == IMPARO_DT_F32) {
        if (mode == 0) IMPARO_CONV(float, 0); else if (mode == 1) IMPARO_CONV(float, 1); else IMPARO_CONV(float, 2);
    } else if (dtype == IMPARO_DT_BF16) {
        const bool wide = parts == 0 && n_tok >= 64 && (width & 7) == 0 && (((uintptr_t)bcx | (uintptr_t)y) & 15) == 0;
        if (wide) {
            const size_t n8 = (size_t)n_tok * (width >> 3);
            const dim3 g8((unsigned)((n8 + threads - 1) / threads));
            const bool w16 = (((uintptr_t)w) & 15) == 0;         // the fixed-taps versions read the weights 16 bytes at a time
#define IMPARO_CONV8(TAPS_) launch(gated_conv_bf16x8_kernel<TAPS_>, g8, dim3(threads), 0, stream, (const __nv_bfloat16*)bcx, w, bias, \
                   state, item_row_start, item_of_token, item_slot, (__nv_bfloat16*)y, n_tok, width, taps, n_slots, status)
            if (w16 && taps == 2) IMPARO_CONV8(2);
            else if (w16 && taps == 3) IMPARO_CONV8(3);
            else if (w16 && taps == 4) IMPARO_CONV8(4);
            else IMPARO_CONV8(0);
#undef IMPARO_CONV8
        } else if (mode == 0) IMPARO_CONV(__nv_bfloat16, 0);
        else if (mode == 1) IMPARO_CONV(__nv_bfloat16, 1);
        else IMPARO_CONV(__nv_bfloat16, 2);
#undef IMPARO_CONV
    } else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}
