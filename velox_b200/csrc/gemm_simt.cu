// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]): the plain matrix product.
//
// Multiply-adds on the CUDA cores in float32, no tensor cores, no reduced
// precision mode: this is the matrix product of the 32-bit path, and the
// reference against which the tensor-core products are checked.  Every output
// element is the sum over k in ascending order, so a row's result does not
// depend on how many rows the call has.  Any M, N, K.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
gemm_nt_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, const float* __restrict__ bias,
                    TC* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    pdl_wait();
    pdl_trigger();
    __shared__ float As[GS_BK][GS_BM + 1];
    __shared__ float Ws[GS_BK][GS_BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int lk = tid & 15, lr = tid >> 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
        const int k = k0 + lk;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lr + 16 * i;
            const int m = m0 + r, n = n0 + r;
            As[lk][r] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk][r] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty + 16 * i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            C[(size_t)m * ldc + n] = from_f32<TC>(v);
        }
    }
}

// in_dtype: element type of A and W; out_dtype: element type of C.
extern "C" int vx_gemm_nt_simt(const void* A, const void* W, const float* bias, void* C, int M, int N,
                               int K, int lda, int ldw, int ldc, int in_dtype, int out_dtype,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VX_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return VX_ERR_SHAPE;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    if (grid.y > 65535) return VX_ERR_LIMIT;
    if (in_dtype == VX_F32 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_GEMM, (gemm_nt_simt_kernel<float, float>), grid, 256, 0, stream, (const float*)A, (const float*)W, bias, (float*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == VX_BF16 && out_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_GEMM, (gemm_nt_simt_kernel<bf16, bf16>), grid, 256, 0, stream, (const bf16*)A, (const bf16*)W, bias, (bf16*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == VX_BF16 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_GEMM, (gemm_nt_simt_kernel<bf16, float>), grid, 256, 0, stream, (const bf16*)A, (const bf16*)W, bias, (float*)C, M, N, K, lda, ldw, ldc);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
