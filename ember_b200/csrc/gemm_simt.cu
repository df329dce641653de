// C[M,N] = A[M,K] . W[N,K]^T with fp32 FMA on the SIMT pipes, any sizes.
//
// This is the true 32-bit matrix product of the float32 path (no tensor cores, no TF32) and
// the fall-back of the bfloat16 path for shapes the tensor-core kernel refuses.  Activations A
// are float or bf16, weights W are float or bf16 independently (a weight stored in 32-bit
// stays so), accumulation is fp32 with k ascending for every output, so a row's result does
// not depend on what else is in the batch.
//
// Epilogues (the reference's are src/backend/cuda/k_gemm.cu:29-53):
//   0 store in the activation dtype      1 store fp32
//   2 add into an fp32 matrix (residual) 3 silu(c[2j]) * c[2j+1] over interleaved gate/up rows
// An optional fp32 bias[N] is added before the epilogue.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw,
                 const float* __restrict__ bias, void* __restrict__ Cv, int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // tx -> columns, ty -> rows
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    // loader mapping: 256 threads fetch 64 rows x 16 k: thread -> (row = id / 4, k = (id % 4) * 4 .. +3)
    const int lrow = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + j][lrow] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.0f;
            Ws[lk + j][lrow] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float c = acc[i][j] + (bias ? bias[n] : 0.0f);
            if (EPI == 0) {
                ((TA*)Cv)[(size_t)m * ldc + n] = from_float<TA>(c);
            } else if (EPI == 1) {
                ((float*)Cv)[(size_t)m * ldc + n] = c;
            } else if (EPI == 2) {
                float* p = (float*)Cv + (size_t)m * ldc + n;
                *p = *p + c;
            } else {
                if ((j & 1) == 0) {  // n even: gate; n + 1: up (same thread, N is even)
                    const float u = acc[i][j + 1] + (bias ? bias[n + 1] : 0.0f);
                    ((TA*)Cv)[(size_t)m * ldc + (n >> 1)] = from_float<TA>(c / (1.0f + expf(-c)) * u);
                }
            }
        }
    }
}

template <typename TA, typename TW>
int launch(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N, int K,
           int epi, cudaStream_t st) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const TA* a = (const TA*)A;
    const TW* w = (const TW*)W;
    switch (epi) {
        case 0: launch_kernel(gemm_simt_kernel<TA, TW, 0>, grid, 256, 0, st, a, lda, w, ldw, bias, C, ldc, M, N, K); break;
        case 1: launch_kernel(gemm_simt_kernel<TA, TW, 1>, grid, 256, 0, st, a, lda, w, ldw, bias, C, ldc, M, N, K); break;
        case 2: launch_kernel(gemm_simt_kernel<TA, TW, 2>, grid, 256, 0, st, a, lda, w, ldw, bias, C, ldc, M, N, K); break;
        case 3: launch_kernel(gemm_simt_kernel<TA, TW, 3>, grid, 256, 0, st, a, lda, w, ldw, bias, C, ldc, M, N, K); break;
        default: return fail("gemm: unknown epilogue %d", epi);
    }
    return check_launch("gemm_simt");
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_gemm_simt(const void* A, int a_dtype, int lda, const void* W, int w_dtype, int ldw,
                              const float* bias, void* C, int ldc, int M, int N, int K, int epilogue, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fail("gemm: K=%d", K);
    if (lda < K || ldw < K) return fail("gemm: row strides (%d, %d) smaller than K=%d", lda, ldw, K);
    if (epilogue == 3 && (N & 1)) return fail("gemm: the gated epilogue needs an even N, got %d", N);
    if (ldc < (epilogue == 3 ? N / 2 : N)) return fail("gemm: output stride %d too small for N=%d", ldc, N);
    if ((M + BM - 1) / BM > 65535) return fail("gemm: M=%d is too large for one launch", M);
    cudaStream_t st = (cudaStream_t)stream;
    if (a_dtype == EMBER_F32 && w_dtype == EMBER_F32)
        return launch<float, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    if (a_dtype == EMBER_F32 && w_dtype == EMBER_BF16)
        return launch<float, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    if (a_dtype == EMBER_BF16 && w_dtype == EMBER_F32)
        return launch<__nv_bfloat16, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    if (a_dtype == EMBER_BF16 && w_dtype == EMBER_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, M, N, K, epilogue, st);
    return fail("gemm: unsupported dtypes %d/%d", a_dtype, w_dtype);
}
