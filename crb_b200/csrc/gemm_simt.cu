// Plain float32 GEMM on the CUDA cores:  C = alpha * A * op(B) + beta * C  (row-major).
//
// Used where the reference multiplies in full float32 (TF32 is switched off there,
// bigptq.py:11-12) and the contraction is short (K = 128): the trailing update
// W[:, i2:] -= Err @ U[i1:i2, i2:] (bigptq.py:264) and the panel / trailing products of the
// blocked factorisation.  128x128 tile per CTA, 8x8 outputs per thread, K staged through
// shared memory 16 at a time with the next stage prefetched into registers.
#include "common.cuh"

namespace crb {

constexpr int BM = 128, BN = 128, BK = 16;

// TRANS_B = false: B is [K, N] row-major.  TRANS_B = true: B is [N, K] row-major (C += A * B^T).
// LOWER_ONLY: skip tiles that lie strictly above the diagonal (for symmetric rank-k updates).
template <bool TRANS_B, bool LOWER_ONLY>
__global__ void __launch_bounds__(256)
k_sgemm(int M, int N, int K, float alpha, const float* __restrict__ A, int64_t lda,
        const float* __restrict__ B, int64_t ldb, float beta, float* __restrict__ C, int64_t ldc) {
    if (LOWER_ONLY && blockIdx.x > blockIdx.y) return;
    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    // global -> register staging: A tile 128 x 16 = 512 float4, two per thread (k contiguous)
    const int a_row = tid >> 2, a_k4 = (tid & 3) * 4;           // rows a_row and a_row + 64
    // B tile: not transposed 16 x 128 (n contiguous) / transposed 128 x 16 (k contiguous)
    const int b_k = tid >> 5, b_n4 = (tid & 31) * 4;            // rows b_k and b_k + 8
    float4 ra[2], rb[2];

    auto fetch = [&](int k0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = m0 + a_row + 64 * h;
            ra[h] = (m < M) ? *reinterpret_cast<const float4*>(A + (int64_t)m * lda + k0 + a_k4)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
            if (TRANS_B) {
                const int n = n0 + a_row + 64 * h;
                rb[h] = (n < N) ? *reinterpret_cast<const float4*>(B + (int64_t)n * ldb + k0 + a_k4)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                const int n = n0 + b_n4;
                rb[h] = (n < N) ? *reinterpret_cast<const float4*>(B + (int64_t)(k0 + b_k + 8 * h) * ldb + n)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = a_row + 64 * h;
            As[buf][a_k4 + 0][m] = ra[h].x; As[buf][a_k4 + 1][m] = ra[h].y;
            As[buf][a_k4 + 2][m] = ra[h].z; As[buf][a_k4 + 3][m] = ra[h].w;
            if (TRANS_B) {
                Bs[buf][a_k4 + 0][m] = rb[h].x; Bs[buf][a_k4 + 1][m] = rb[h].y;
                Bs[buf][a_k4 + 2][m] = rb[h].z; Bs[buf][a_k4 + 3][m] = rb[h].w;
            } else {
                *reinterpret_cast<float4*>(&Bs[buf][b_k + 8 * h][b_n4]) = rb[h];
            }
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    fetch(0);
    stash(0);
    __syncthreads();
    const int nk = K / BK;
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) fetch((kt + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4 + 64]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4 + 64]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            stash(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + ty * 4 + (i & 3) + 64 * (i >> 2);
        if (m >= M) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = n0 + tx * 4 + 64 * h;
            if (n >= N) continue;
            float4* p = reinterpret_cast<float4*>(C + (int64_t)m * ldc + n);
            float4 c = (beta != 0.f) ? *p : make_float4(0.f, 0.f, 0.f, 0.f);
            c.x = fmaf(alpha, acc[i][4 * h + 0], beta * c.x);
            c.y = fmaf(alpha, acc[i][4 * h + 1], beta * c.y);
            c.z = fmaf(alpha, acc[i][4 * h + 2], beta * c.z);
            c.w = fmaf(alpha, acc[i][4 * h + 3], beta * c.w);
            *p = c;
        }
    }
}

// C[M,N] = alpha * A[M,K] * op(B) + beta * C.  Requirements: K % 16 == 0, N % 4 == 0, all
// leading dimensions % 4 == 0 and base pointers 16-byte aligned.
int sgemm(bool trans_b, bool lower_only, int M, int N, int K, float alpha, const float* A,
          int64_t lda, const float* B, int64_t ldb, float beta, float* C, int64_t ldc,
          cudaStream_t st) {
    if (M <= 0 || N <= 0) return CRB_OK;
    if (K <= 0 || (K % BK) || (N & 3) || (lda & 3) || (ldb & 3) || (ldc & 3)) return CRB_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return CRB_ERR_BAD_ARG;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (trans_b) {
        if (lower_only) k_sgemm<true, true><<<grid, 256, 0, st>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
        else k_sgemm<true, false><<<grid, 256, 0, st>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
    } else {
        if (lower_only) k_sgemm<false, true><<<grid, 256, 0, st>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
        else k_sgemm<false, false><<<grid, 256, 0, st>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
    }
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
