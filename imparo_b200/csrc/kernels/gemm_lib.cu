// Library matrix product for bfloat16 weights: out[M,N] (+)= A[M,K] * W[N,K]^T through
// cuBLAS with 32-bit accumulation.  The reference's engine also hands its dense
// bfloat16 products to this library (imparo-cuda/native/bf16_bounded_gemm.cuh:4-28).
// The hand-written tcgen05 kernel (gemm_tcgen05.cu) replaces it where it is faster.
#include "common.cuh"
#include <cublas_v2.h>

#ifdef IMPARO_TIMELINE
// The library's kernels carry no stamps: in the timeline build a one-warp kernel of ours follows
// each library product, so that the product's time shows as the share of the kernel before it up
// to this marker and the hand-over to the next kernel as the marker's own.
namespace imparo {
__global__ void library_product_done_kernel() {
    pdl_trigger();
    pdl_wait();
}
}
#endif

namespace {
cublasHandle_t g_handle = nullptr;
void* g_workspace = nullptr;
size_t g_workspace_bytes = 0;
bool g_bound = false;                 // g_handle is set to g_bound_stream and the workspace
cudaStream_t g_bound_stream = nullptr;
}

// workspace: device memory the caller owns for as long as products run (stable address,
// so captured graphs stay valid).
extern "C" int imparo_gemm_lib_init(void* workspace, size_t workspace_bytes) {
    if (!g_handle) {
        cublasStatus_t s = cublasCreate(&g_handle);
        if (s != CUBLAS_STATUS_SUCCESS) return 1000 + (int)s;
    }
    g_workspace = workspace;
    g_workspace_bytes = workspace_bytes;
    g_bound = false;
    return 0;
}

// c_dtype: 0 = float32 out, 1 = bfloat16 out.  accumulate adds into C (32-bit C only).
extern "C" int imparo_gemm_bf16_nt(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K,
                                   int lda, int ldc, int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!g_handle) return -1;
    if (accumulate && c_dtype != IMPARO_DT_F32) return -2;
    cublasStatus_t s;
    if (!g_bound || g_bound_stream != stream) {
        // setting the stream resets the library's workspace to its own, so both are set together,
        // and only when the stream changes (a step issues dozens of products on one stream)
        s = cublasSetStream(g_handle, stream);
        if (s != CUBLAS_STATUS_SUCCESS) return 1000 + (int)s;
        if (g_workspace) {
            s = cublasSetWorkspace(g_handle, g_workspace, g_workspace_bytes);
            if (s != CUBLAS_STATUS_SUCCESS) return 1000 + (int)s;
        }
        g_bound = true;
        g_bound_stream = stream;
    }
    const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
    // column-major view: C^T[N,M] = W[N,K] * A^T[K,M]
    s = cublasGemmEx(g_handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha,
                     W, CUDA_R_16BF, K, A, CUDA_R_16BF, lda, &beta,
                     C, c_dtype == IMPARO_DT_F32 ? CUDA_R_32F : CUDA_R_16BF, ldc,
                     CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (s != CUBLAS_STATUS_SUCCESS) return 1000 + (int)s;
#ifdef IMPARO_TIMELINE
    launch(imparo::library_product_done_kernel, dim3(1), dim3(32), 0, stream);
#endif
    return 0;
}
