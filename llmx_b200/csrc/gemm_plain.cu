// Plain matrix product on the CUDA cores: C[M, N] (+)= A[M, K] * W[N, K]^T.
//
// This is the product of the true 32-bit path (32-bit inputs, explicit fmaf, no
// reduced-precision matrix mode) and the fallback of the bfloat16 path for widths a
// TMA descriptor cannot take (a row stride that is not a multiple of 16 bytes).
// Each output's sum runs over k in increasing order whatever M is, so a row's result
// does not depend on what else is in the batch (the reference's rule,
// src/backends/backend.hpp:141-150; its kernels: f32.gpu:1034-1084).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

template <typename AT, typename WT>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const AT* __restrict__ A, const WT* __restrict__ W,
                                                         float* __restrict__ C, int M, int N, int K, int accumulate) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements per operand, 256 threads: four each, consecutive k fastest.
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int e = threadIdx.x + it * 256;
            const int r = e >> 4, k = e & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * K + gk]) : 0.0f;
            Ws[k][r] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float* c = C + (size_t)gm * N + gn;
            *c = accumulate ? *c + acc[i][j] : acc[i][j];
        }
    }
}
}  // namespace

LLMX_EXPORT int llmx_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, float* C, int M, int N, int K,
                                int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return LLMX_ERR_BAD_ARGUMENT;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return LLMX_ERR_UNSUPPORTED;
    if (a_dtype == LLMX_F32 && w_dtype == LLMX_F32)
        launch_kernel(gemm_plain_kernel<float, float>, dim3(grid), dim3(256), 0, stream, (const float*)A, (const float*)W, C, M, N, K, accumulate);
    else if (a_dtype == LLMX_BF16 && w_dtype == LLMX_BF16)
        launch_kernel(gemm_plain_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, C, M, N, K, accumulate);
    else
        return LLMX_ERR_UNSUPPORTED;
    return launch_status();
}
