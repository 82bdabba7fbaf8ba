// True 32-bit matrix product: out[M,N] (+)= A[M,K] * W[N,K]^T, FFMA only.
//
// This is the matrix product of the 32-bit path: no tensor cores, no reduced-precision
// mode.  Every output element is one accumulator summed over k = 0..K-1 in order, so a
// row's result does not depend on how many other rows the call carries.  Layout follows
// the reference: W[n_out, n_in] row-major, y[t,o] = sum_i W[o,i]*x[t,i]
// (imparo-cpu/src/ops.rs:660,688-690).
#include "common.cuh"

namespace imparo {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldc, int accumulate) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;        // 16 x 16 threads, each 4 x 4 outputs
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // each thread loads 4 elements of each tile: row = idx / BK, col = idx % BK
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 256;
            const int row = idx / BK, col = idx % BK;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + col;
            As[col][row] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[col][row] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float* c = C + (size_t)gm * ldc + gn;
            *c = accumulate ? (*c + acc[i][j]) : acc[i][j];
        }
    }
}

}  // namespace imparo

extern "C" int imparo_sgemm_nt(const float* A, const float* W, float* C, int M, int N, int K,
                               int lda, int ldc, int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return -1;
    dim3 grid((N + imparo::BN - 1) / imparo::BN, (M + imparo::BM - 1) / imparo::BM);
    if (grid.y > 65535) return -2;
    launch(imparo::sgemm_nt_kernel, grid, dim3(256), 0, stream, A, W, C, M, N, K, lda, ldc, accumulate);
    IMPARO_CHECK_LAUNCH();
    return 0;
}
