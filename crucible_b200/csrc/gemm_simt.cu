// C[M,N] (+)= A[M,K] . W[N,K]^T on CUDA cores with fp32 multiply-add: the
// matrix product of the true 32-bit path, and the refuge of the bfloat16 path
// for shapes its tensor-core kernel refuses.  No tensor cores, no reduced-
// precision mode.  Every output element is one sum over k in ascending order,
// whatever M and N are and wherever its tile lies, so a row's result does not
// depend on what else is in the batch.
//
// Reference counterpart: `gemm_f32` (engine/kernels/kernels.cu:922), 16x16
// scalar tiles; this one uses 64x64 tiles with a 4x4 micro-tile per thread.
#define CB_PDL_BIT 9      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TA, typename TC, bool ACCUMULATE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, TC* __restrict__ C,
                 int M, int N, int K, int lda, int ldw, int ldc) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float As[TK][TM + 4];
    __shared__ float Ws[TK][TN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;           // 16 x 16 threads, 4 x 4 each
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f;
            if (k < K) {
                if (m0 + r < M) a = cb_to_float(A[(size_t)(m0 + r) * lda + k]);
                if (n0 + r < N) w = cb_to_float(W[(size_t)(n0 + r) * ldw + k]);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            TC* p = C + (size_t)m * ldc + n;
            if (ACCUMULATE) *p = cb_from_float<TC>(cb_to_float(*p) + acc[i][j]);
            else *p = cb_from_float<TC>(acc[i][j]);
        }
    }
}

template <typename TA, typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw,
           int ldc, int accumulate, cudaStream_t s) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (accumulate)
        cb_launch(gemm_simt_kernel<TA, TC, true>, dim3(grid), dim3(256), 0, s, (const TA*)A, (const TA*)W, (TC*)C,
                                                            M, N, K, lda, ldw, ldc);
    else
        cb_launch(gemm_simt_kernel<TA, TC, false>, dim3(grid), dim3(256), 0, s, (const TA*)A, (const TA*)W, (TC*)C,
                                                             M, N, K, lda, ldw, ldc);
    return cb_last_error();
}

}  // namespace

// in_dtype: dtype of A and W; out_dtype: dtype of C.  accumulate: C += A.W^T.
CB_EXPORT int cb_gemm_simt(const void* A, const void* W, void* C, int in_dtype, int out_dtype,
                           int M, int N, int K, int lda, int ldw, int ldc, int accumulate,
                           void* stream) {
    if (M <= 0 || N <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == CB_F32 && out_dtype == CB_F32)
        return launch<float, float>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, s);
    if (in_dtype == CB_BF16 && out_dtype == CB_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, s);
    if (in_dtype == CB_BF16 && out_dtype == CB_F32)
        return launch<__nv_bfloat16, float>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, s);
    return CB_ERR_UNSUPPORTED;
}
