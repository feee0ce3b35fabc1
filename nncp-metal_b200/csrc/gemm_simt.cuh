// gemm_simt.cuh -- CUDA-core GEMM with fp32 accumulation.
//
// The fp32 engine of the library (fp32 models must not lose mantissa bits to
// tensor-core input formats) and the reference every tensor-core kernel is
// checked against.  Replaces nc_matmul / nc_matmul_add (libnc.h:270-276).
//
// Every output element is one fp32 accumulator that receives fmaf(a, b, acc)
// for k = 0, 1, ... K-1 in that order, whatever the tile shape or the number
// of rows in the launch: a row computed alone (one-symbol step) is bit-identical
// to the same row computed inside a whole segment.
#pragma once
#include "common.cuh"

enum { GEMM_NT = 0, GEMM_NN = 1, GEMM_TN = 2 };
// NT: C[m][n] = sum_k A[m][k] * B[n][k]      (y = x W^T)
// NN: C[m][n] = sum_k A[m][k] * B[k][n]      (dx = dy W)
// TN: C[m][n] = sum_k A[k][m] * B[k][n]      (dW = dy^T x; k runs over rows)

template <int BM, int BN, int TM, int TN, int MODE, typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(int M, int N, int K, const TA *__restrict__ A, long lda,
                 const TB *__restrict__ B, long ldb, TC *__restrict__ C, long ldc,
                 const float *__restrict__ bias, int accumulate, int bias_n)
{
    constexpr int BK = 16;
    constexpr int LDAS = BM + 4, LDBS = BN + 4;
    static_assert((BM / TM) * (BN / TN) == 256, "256 threads per tile");
    static_assert(TM % 4 == 0 && TN % 4 == 0, "register tile in float4 units");
    __shared__ __align__(16) float As[BK][LDAS];
    __shared__ __align__(16) float Bs[BK][LDBS];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    constexpr int CM = TM / 4, CN = TN / 4; // float4 chunks per thread
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++)
            acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        if (MODE == GEMM_TN) { // A[k][m], m contiguous
            for (int e = tid; e < BM * BK; e += 256) {
                int m = e % BM, k = e / BM;
                int gm = m0 + m, gk = k0 + k;
                As[k][m] = (gm < M && gk < K) ? to_f(A[(long)gk * lda + gm]) : 0.0f;
            }
        } else { // A[m][k], k contiguous
            for (int e = tid; e < BM * BK; e += 256) {
                int k = e % BK, m = e / BK;
                int gm = m0 + m, gk = k0 + k;
                As[k][m] = (gm < M && gk < K) ? to_f(A[(long)gm * lda + gk]) : 0.0f;
            }
        }
        if (MODE == GEMM_NT) { // B[n][k], k contiguous
            for (int e = tid; e < BN * BK; e += 256) {
                int k = e % BK, n = e / BK;
                int gn = n0 + n, gk = k0 + k;
                Bs[k][n] = (gn < N && gk < K) ? to_f(B[(long)gn * ldb + gk]) : 0.0f;
            }
        } else { // B[k][n], n contiguous
            for (int e = tid; e < BN * BK; e += 256) {
                int n = e % BN, k = e / BN;
                int gn = n0 + n, gk = k0 + k;
                Bs[k][n] = (gn < N && gk < K) ? to_f(B[(long)gk * ldb + gn]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM], b[TN];
#pragma unroll
            for (int c = 0; c < CM; c++) {
                float4 v = *reinterpret_cast<const float4 *>(&As[k][c * (BM / CM) + ty * 4]);
                a[c * 4 + 0] = v.x; a[c * 4 + 1] = v.y; a[c * 4 + 2] = v.z; a[c * 4 + 3] = v.w;
            }
#pragma unroll
            for (int c = 0; c < CN; c++) {
                float4 v = *reinterpret_cast<const float4 *>(&Bs[k][c * (BN / CN) + tx * 4]);
                b[c * 4 + 0] = v.x; b[c * 4 + 1] = v.y; b[c * 4 + 2] = v.z; b[c * 4 + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++)
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        int gm = m0 + (i / 4) * (BM / CM) + ty * 4 + (i % 4);
        if (gm >= M)
            continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            int gn = n0 + (j / 4) * (BN / CN) + tx * 4 + (j % 4);
            if (gn >= N)
                continue;
            float v = acc[i][j];
            if (bias && gn < bias_n)
                v += bias[gn];
            TC *dst = C + (long)gm * ldc + gn;
            if (accumulate)
                v += to_f(*dst);
            *dst = from_f<TC>(v);
        }
    }
}

template <int MODE, typename TA, typename TB, typename TC>
static int gemm_simt_mode(cudaStream_t st, int M, int N, int K, const TA *A, long lda,
                          const TB *B, long ldb, TC *C, long ldc, const float *bias, int acc, int bias_n)
{
    long big_tiles = (long)ceil_div(M, 128) * ceil_div(N, 128);
    if (big_tiles >= 96) {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 128));
        gemm_simt_kernel<128, 128, 8, 8, MODE, TA, TB, TC>
            <<<grid, 256, 0, st>>>(M, N, K, A, lda, B, ldb, C, ldc, bias, acc, bias_n);
    } else {
        dim3 grid(ceil_div(N, 64), ceil_div(M, 64));
        gemm_simt_kernel<64, 64, 4, 4, MODE, TA, TB, TC>
            <<<grid, 256, 0, st>>>(M, N, K, A, lda, B, ldb, C, ldc, bias, acc, bias_n);
    }
    KERNEL_CHECK();
    return NNCU_OK;
}

template <typename TA, typename TB, typename TC>
static int gemm_simt(cudaStream_t st, int mode, int M, int N, int K, const TA *A, long lda,
                     const TB *B, long ldb, TC *C, long ldc, const float *bias, int acc, int bias_n = 1 << 30)
{
    if (M <= 0 || N <= 0)
        return NNCU_OK;
    switch (mode) {
    case GEMM_NT: return gemm_simt_mode<GEMM_NT>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, acc, bias_n);
    case GEMM_NN: return gemm_simt_mode<GEMM_NN>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, acc, bias_n);
    case GEMM_TN: return gemm_simt_mode<GEMM_TN>(st, M, N, K, A, lda, B, ldb, C, ldc, bias, acc, bias_n);
    }
    return nncu_fail(NNCU_ERR_INVALID, "gemm_simt: bad mode %d", mode);
}
