// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the FP32 cores: the matrix product
// of the true 32-bit path (no tensor cores, hence no reduced-precision matrix
// mode), and a fallback of the bf16 path for sizes the tensor-core kernel
// refuses.  Every output element is the sum over k = 0..K-1 in that order,
// whatever M is and wherever the element lies in its tile, so a row's result
// does not depend on what else is in the batch.
//
// y = x W^T + b with W stored [out, in]:
// crane-core/src/models/hunyuan_dense/modeling.rs:273-330.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, const float* __restrict__ bias,
               TO* __restrict__ C, int M, int N, int K, long long lda, long long ldw,
               long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of A and 4 of W per k-slab: row = tid / 4, 4 k's
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lr, n = n0 + lr;
            As[lk + i][lr] = (m < M && k < K) ? to_f32(A[(long long)m * lda + k]) : 0.f;
            Ws[lk + i][lr] = (n < N && k < K) ? to_f32(W[(long long)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            C[(long long)m * ldc + n] = from_f32<TO>(v);
        }
    }
}
}  // namespace

// in_dtype / out_dtype: 0 = float, 1 = bf16 (out may be float with bf16 inputs).
CRANE_API int crane_gemm_simt(int in_dtype, int out_dtype, const void* A, const void* W,
                              const float* bias, void* C, int M, int N, int K, long long lda,
                              long long ldw, long long ldc, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (in_dtype == 0 && out_dtype == 0)
        gemm_nt_kernel<float, float><<<grid, 256, 0, st>>>((const float*)A, (const float*)W, bias,
                                                           (float*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == 1 && out_dtype == 1)
        gemm_nt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(
            (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (__nv_bfloat16*)C, M, N, K,
            lda, ldw, ldc);
    else if (in_dtype == 1 && out_dtype == 0)
        gemm_nt_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(
            (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (float*)C, M, N, K, lda, ldw,
            ldc);
    else
        return (int)cudaErrorInvalidValue;
    return crane_launch_status();
}
