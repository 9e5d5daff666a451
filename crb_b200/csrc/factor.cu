// Damping and the inverse factor  U = chol(inv(H), upper)  entirely on the device.
// Replaces bigptq.py:101-129 (dead columns, percdamp * mean(diag) damping, cholesky ->
// cholesky_inverse -> cholesky(upper)).
//
// Identity used: if H = V V^T with V upper triangular, then inv(H) = V^-T V^-1, so the upper
// factor with inv(H) = U^T U is U = V^-1.  V is obtained from an ordinary lower Cholesky
// factorisation of the index-reversed matrix (H_r[i][j] = H[C-1-i][C-1-j] = L L^T gives
// V = reverse(L)), so U = reverse(L^-1): one factorisation and one triangular inverse
// (2 C^3 / 3 flop) instead of the reference's three library calls (4 C^3 / 3 flop).
//
// Blocked at two levels.  Per 128-wide diagonal block: one CTA factors the 128x128 block in
// shared memory and inverts it; the rows below are multiplied by that inverse and the rest of
// the current 1024-wide outer panel gets a rank-128 update.  After the panel's last block the
// whole trailing matrix is updated once with K = 1024.  All products run through the split-TF32
// tensor-core GEMM (gemm_tc.cu).  The triangular inverse merges neighbouring diagonal blocks
// recursively: [[A,0],[B,D]]^-1 = [[A^-1,0],[-D^-1 B A^-1, D^-1]], skipping the zero halves.
// A non-positive pivot sets CRB_FLAG_BAD_PIVOT (the host re-damps and calls again, like the
// retry loop at bigptq.py:115-123) and is replaced by 1 so that nothing non-finite spreads.
#include <map>
#include <utility>
#include <vector>

#include "common.cuh"

namespace crb {

constexpr int FB = 128;    // panel width
constexpr int kOuter = 8;  // diagonal blocks per outer panel of the factorisation

// diag statistics: dead columns, mean of the diagonal after the dead fix, total damping.
__global__ void __launch_bounds__(1024)
k_diag_prepare(const float* __restrict__ H, int C, float percdamp, int extra_steps,
               float* __restrict__ damp_out, unsigned char* __restrict__ dead) {
    __shared__ double s_part[32];
    double s = 0.0;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
        float d = H[(int64_t)i * C + i];
        const bool is_dead = (d == 0.f);
        dead[i] = is_dead;
        if (is_dead) d = 1.f;
        s += (double)d;
    }
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
        float mean = (float)(tot / C);
        float damp = percdamp * mean;              // bigptq.py:109-111
        mean += damp;
        for (int k = 0; k < extra_steps; ++k) {    // bigptq.py:120-123, one step per failed attempt
            float extra = 1e-3f * mean;
            if (extra == 0.f) extra = 1e-6f;
            damp += extra;
            mean += extra;
        }
        *damp_out = damp;
    }
}

__global__ void k_zero_dead(float* __restrict__ W, int R, int C, int64_t ldw,
                            const unsigned char* __restrict__ dead) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C || !dead[c]) return;
    for (int r = blockIdx.y; r < R; r += gridDim.y) W[(int64_t)r * ldw + c] = 0.f;   // bigptq.py:105
}

// A = index-reversed copy of the damped H (lower triangle and diagonal; zeros above).
__global__ void k_reverse_copy(const float* __restrict__ H, int C, const float* __restrict__ damp,
                               const unsigned char* __restrict__ dead, float* __restrict__ A) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = blockIdx.y;
    if (j >= C) return;
    float v = 0.f;
    if (j <= i) {
        const int si = C - 1 - i, sj = C - 1 - j;
        v = H[(int64_t)si * C + sj];
        if (i == j) v = (dead[si] ? 1.f : v) + *damp;
    }
    A[(int64_t)i * C + j] = v;
}

// Factor one 128x128 diagonal block (lower Cholesky) and overwrite it with the inverse of its
// factor (zeros above the diagonal).  One CTA of 512 threads, blocked by 16 columns:
//   phase 1, per 16-column panel: one warp factors the 16x16 diagonal block and inverts it with
//            shuffles; the rows below are multiplied by that inverse; the trailing block gets a
//            rank-16 update with 4x4 register tiles (16-byte shared-memory loads);
//   phase 2: the inverse is assembled from the 16x16 diagonal inverses by merging neighbouring
//            blocks three times:  [[A,0],[B,D]]^-1 = [[A^-1,0],[-D^-1 B A^-1, D^-1]].
constexpr int kDiagThreads = 512;
constexpr int kDiagPitch = FB + 4;                 // 132 floats: rows 16-byte aligned, 8 rows hit 8 bank groups
constexpr int kDiagTmpPitch = 68;
constexpr int kLiPitch = 20;                       // rows of the 16x16 inverse: 16-byte aligned
constexpr int kDiagSmemFloats = 2 * FB * kDiagPitch + 64 * kDiagTmpPitch;

// C[i][j] (+)= sign * sum_k A[i][k] * B[k][j] for an n x n block, 4x4 outputs per thread, rows and
// columns of a thread's tile strided by n/4 so that consecutive lanes read consecutive rows.
template <bool SUBTRACT_FROM_ZERO>
__device__ __forceinline__ void smem_gemm_nn(const float* A, int lda, const float* B, int ldb, float* C, int ldc,
                                             int n, int tid_in_group, int group_threads) {
    const int q = n >> 2;                           // tile grid q x q, strided rows / contiguous 4-column groups
    for (int idx = tid_in_group; idx < q * q; idx += group_threads) {
        const int ti = idx % q, tj = idx / q;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
        for (int k = 0; k < n; k += 4) {
            float4 av[4], bv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) av[a] = *reinterpret_cast<const float4*>(A + (ti + a * q) * lda + k);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) bv[kk] = *reinterpret_cast<const float4*>(B + (k + kk) * ldb + 4 * tj);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float ak[4] = {av[a].x, av[a].y, av[a].z, av[a].w};
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    acc[a][0] = fmaf(ak[kk], bv[kk].x, acc[a][0]);
                    acc[a][1] = fmaf(ak[kk], bv[kk].y, acc[a][1]);
                    acc[a][2] = fmaf(ak[kk], bv[kk].z, acc[a][2]);
                    acc[a][3] = fmaf(ak[kk], bv[kk].w, acc[a][3]);
                }
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            float4 o = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
            if (SUBTRACT_FROM_ZERO) { o.x = -o.x; o.y = -o.y; o.z = -o.z; o.w = -o.w; }
            *reinterpret_cast<float4*>(C + (ti + a * q) * ldc + 4 * tj) = o;
        }
    }
}

// Waits (bounded) until a shared-memory progress counter has reached `need`; false if it gave up.
__device__ __forceinline__ bool wait_progress(volatile int* counter, int need) {
    for (int it = 0; it < (1 << 22); ++it) {
        if (*counter >= need) { __threadfence_block(); return true; }
    }
    return false;
}

__global__ void __launch_bounds__(kDiagThreads)
k_chol_diag(float* __restrict__ Akk, int64_t ld, unsigned* status) {
    extern __shared__ __align__(16) float s_diag[];
    float* a = s_diag;                               // [128][132] the block, then its factor L
    float* x = s_diag + FB * kDiagPitch;             // [128][132] the inverse of L
    float* tmp = x + FB * kDiagPitch;                // [64][68]   products of phase 2
    __shared__ __align__(16) float s_li[2][16][kLiPitch];   // inverse of the 16x16 diagonal factor of step j (buffer j & 1)
    __shared__ int s_bad, s_gave_up;
    __shared__ volatile int s_crit;                  // steps whose diagonal block AND look-ahead row are done (warp 0)
    __shared__ volatile int s_bulk;                  // steps whose panel + trailing update are done (warps 1..15)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { s_bad = 0; s_gave_up = 0; s_crit = 0; s_bulk = 0; }
    chain_wait();
    {
        // 16-byte loads, all eight of a thread in flight before the first store
        float4 v[FB * FB / 4 / kDiagThreads];
#pragma unroll
        for (int u = 0; u < FB * FB / 4 / kDiagThreads; ++u) {
            const int e = 4 * (tid + u * kDiagThreads);
            v[u] = *reinterpret_cast<const float4*>(Akk + (int64_t)(e >> 7) * ld + (e & 127));
        }
#pragma unroll
        for (int u = 0; u < FB * FB / 4 / kDiagThreads; ++u) {
            const int e = 4 * (tid + u * kDiagThreads);
            *reinterpret_cast<float4*>(a + (e >> 7) * kDiagPitch + (e & 127)) = v[u];
            *reinterpret_cast<float4*>(x + (e >> 7) * kDiagPitch + (e & 127)) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    __syncthreads();

    // ---------------- phase 1: blocked Cholesky, 16 columns per step ----------------
    // The chain that cannot be parallelised is: factor and invert the 16x16 diagonal block of step
    // j, then bring the NEXT 16 rows up to date so that step j + 1 can start.  Warp 0 does exactly
    // that and runs ahead; warps 1..15 follow one step behind with the rest of step j's work (the
    // panel below those 16 rows and the rank-16 update of the trailing block).  Every element still
    // receives the same updates in the same order as in a step-by-step factorisation.
    constexpr int kSteps = FB / 16;
    constexpr int kBulkThreads = kDiagThreads - 32;
    if (warp == 0) {
        for (int j = 0; j < kSteps; ++j) {
            const int c0 = 16 * j;
            float (*li)[kLiPitch] = s_li[j & 1];
            {
                // 16x16 diagonal block: lane i (and its mirror i + 16) holds row i of the block and
                // column i of the inverse.  This warp is the serial core of the whole factorisation
                // (a timeline of the kernel showed 6 us per step here with IEEE sqrt and divisions
                // in the chain against 1 us for everything else), so the pivots go through
                // rsqrt + one Newton step and the inverse rows are produced inside the same loop:
                // row k of the inverse only needs rows < k of it and row k of L, which is final once
                // column k has been scaled, and its chain runs beside the update of the block.
                const int i = lane & 15;
                float d[16], xi[16];
#pragma unroll
                for (int jj = 0; jj < 16; jj += 4) {
                    const float4 v = *reinterpret_cast<const float4*>(a + (c0 + i) * kDiagPitch + c0 + jj);
                    d[jj] = v.x; d[jj + 1] = v.y; d[jj + 2] = v.z; d[jj + 3] = v.w;
                }
                bool bad = false;
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    float piv = __shfl_sync(0xffffffffu, d[k], k);
                    if (!(piv > 0.f) || !isfinite(piv)) { bad = true; piv = 1.f; }
                    float rs = rsqrtf(piv);
                    rs = rs * fmaf(-0.5f * piv * rs, rs, 1.5f);           // 1 / sqrt(piv) to float32 accuracy
                    const float lik = (i == k) ? piv * rs : d[k] * rs;    // L[i][k] (rows i >= k meaningful)
                    d[k] = lik;
                    // row k of the inverse: X[k][i] = ((k == i) - sum_{m<k} L[k][m] X[m][i]) / L[k][k];
                    // rows above the diagonal come out as exact zeros
                    float acc = (k == i) ? 1.f : 0.f;
#pragma unroll
                    for (int m = 0; m < k; ++m) acc = fmaf(-__shfl_sync(0xffffffffu, d[m], k), xi[m], acc);
                    xi[k] = acc * rs;
#pragma unroll
                    for (int jj = k + 1; jj < 16; ++jj)
                        d[jj] = fmaf(-lik, __shfl_sync(0xffffffffu, lik, jj), d[jj]);   // used only for i >= jj
                }
                if (bad && lane == 0) s_bad = 1;
                if (lane < 16) {
#pragma unroll
                    for (int jj = 0; jj < 16; jj += 4)
                        *reinterpret_cast<float4*>(a + (c0 + i) * kDiagPitch + c0 + jj) =
                            make_float4(jj <= i ? d[jj] : 0.f, jj + 1 <= i ? d[jj + 1] : 0.f, jj + 2 <= i ? d[jj + 2] : 0.f,
                                        jj + 3 <= i ? d[jj + 3] : 0.f);
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        li[r][i] = xi[r];
                        x[(c0 + r) * kDiagPitch + c0 + i] = xi[r];
                    }
                }
            }
            __syncwarp();
            if (j + 1 < kSteps) {
                // the next 16 rows have received every update of the steps before j once the other
                // warps are through with step j - 1
                if (lane == 0 && !wait_progress(&s_bulk, j)) s_gave_up = 1;
                __syncwarp();
                // look-ahead: P = A[next 16 rows, this step's columns] * Linv^T (two lanes per row,
                // eight columns each; Linv[col][m] is zero for m > col), then the next diagonal
                // block -= P P^T
                const int r = lane >> 1, h = lane & 1;
                float* prow = a + (c0 + 16 + r) * kDiagPitch + c0;
                float in[16];
#pragma unroll
                for (int m = 0; m < 16; m += 4) {
                    const float4 v = *reinterpret_cast<const float4*>(prow + m);
                    in[m] = v.x; in[m + 1] = v.y; in[m + 2] = v.z; in[m + 3] = v.w;
                }
                __syncwarp();
                float pout[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    const float4* lrow = reinterpret_cast<const float4*>(&li[8 * h + jj][0]);
                    float acc = 0.f;
#pragma unroll
                    for (int m4 = 0; m4 < 4; ++m4) {
                        const float4 v = lrow[m4];
                        acc = fmaf(in[4 * m4], v.x, acc); acc = fmaf(in[4 * m4 + 1], v.y, acc);
                        acc = fmaf(in[4 * m4 + 2], v.z, acc); acc = fmaf(in[4 * m4 + 3], v.w, acc);
                    }
                    pout[jj] = acc;
                }
                *reinterpret_cast<float4*>(prow + 8 * h) = make_float4(pout[0], pout[1], pout[2], pout[3]);
                *reinterpret_cast<float4*>(prow + 8 * h + 4) = make_float4(pout[4], pout[5], pout[6], pout[7]);
                __syncwarp();
                const float* P = a + (c0 + 16) * kDiagPitch + c0;        // P[i][m], 16 x 16
                float* D = a + (c0 + 16) * kDiagPitch + c0 + 16;         // the next diagonal block
                float pr[16];
#pragma unroll
                for (int m = 0; m < 16; m += 4) {
                    const float4 v = *reinterpret_cast<const float4*>(P + r * kDiagPitch + m);
                    pr[m] = v.x; pr[m + 1] = v.y; pr[m + 2] = v.z; pr[m + 3] = v.w;
                }
                float upd[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    const float4* crow = reinterpret_cast<const float4*>(P + (8 * h + jj) * kDiagPitch);
                    float acc = 0.f;
#pragma unroll
                    for (int m4 = 0; m4 < 4; ++m4) {
                        const float4 v = crow[m4];
                        acc = fmaf(pr[4 * m4], v.x, acc); acc = fmaf(pr[4 * m4 + 1], v.y, acc);
                        acc = fmaf(pr[4 * m4 + 2], v.z, acc); acc = fmaf(pr[4 * m4 + 3], v.w, acc);
                    }
                    upd[jj] = acc;
                }
                float4* dst = reinterpret_cast<float4*>(D + r * kDiagPitch + 8 * h);
                float4 o0 = dst[0], o1 = dst[1];
                o0.x -= upd[0]; o0.y -= upd[1]; o0.z -= upd[2]; o0.w -= upd[3];
                o1.x -= upd[4]; o1.y -= upd[5]; o1.z -= upd[6]; o1.w -= upd[7];
                dst[0] = o0; dst[1] = o1;
            }
            __threadfence_block();
            __syncwarp();
            if (lane == 0) s_crit = j + 1;
        }
    } else {
        const int bt = tid - 32;                                       // 0 .. 479
        for (int j = 0; j + 1 < kSteps; ++j) {
            const int c0 = 16 * j;
            if (lane == 0 && !wait_progress(&s_crit, j + 1)) s_gave_up = 1;
            __syncwarp();
            __threadfence_block();
            const float (*li)[kLiPitch] = s_li[j & 1];
            const int below = FB - c0 - 32;                            // rows under the look-ahead rows
            if (below > 0) {
                // panel: P[i][col] = sum_{m <= col} A[i][c0 + m] * Linv[col][m]; four threads share a row
                const int r = bt >> 2, jg = bt & 3;
                const bool act = r < below;
                float* prow = a + (c0 + 32 + (act ? r : 0)) * kDiagPitch + c0;
                float in[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) in[m] = prow[m];
                asm volatile("bar.sync 1, %0;" ::"n"(kBulkThreads) : "memory");
                if (act) {
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int col = 4 * jg + jj;
                        float acc = 0.f;
#pragma unroll
                        for (int m = 0; m < 16; ++m) acc = fmaf(in[m], (m <= col) ? li[col][m] : 0.f, acc);
                        prow[col] = acc;
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kBulkThreads) : "memory");
                // trailing update: rows from c0 + 32 on, columns from c0 + 16 on (the first 16 of them
                // pair with the look-ahead rows of warp 0):  A[i][c] -= sum_m P[i][m] P[c][m]
                const int qi = below >> 2, qj = (below + 16) >> 2;
                const float* P = a + (c0 + 16) * kDiagPitch + c0;       // P of row (c0 + 16 + k) at P[k]
                float* T = a + (c0 + 32) * kDiagPitch + c0 + 16;        // T[i][c]: row c0 + 32 + i, column c0 + 16 + c
                for (int idx = bt; idx < qi * qj; idx += kBulkThreads) {
                    const int ti = idx % qi, tj = idx / qi;
                    if (16 + ti + 3 * qi < 4 * tj) continue;            // tile entirely above the diagonal
                    float acc[4][4];
#pragma unroll
                    for (int aa = 0; aa < 4; ++aa)
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb) acc[aa][bb] = 0.f;
#pragma unroll
                    for (int m = 0; m < 16; m += 4) {
                        float4 pi[4], pj[4];
#pragma unroll
                        for (int aa = 0; aa < 4; ++aa) pi[aa] = *reinterpret_cast<const float4*>(P + (16 + ti + aa * qi) * kDiagPitch + m);
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb) pj[bb] = *reinterpret_cast<const float4*>(P + (4 * tj + bb) * kDiagPitch + m);
#pragma unroll
                        for (int aa = 0; aa < 4; ++aa)
#pragma unroll
                            for (int bb = 0; bb < 4; ++bb) {
                                acc[aa][bb] = fmaf(pi[aa].x, pj[bb].x, acc[aa][bb]);
                                acc[aa][bb] = fmaf(pi[aa].y, pj[bb].y, acc[aa][bb]);
                                acc[aa][bb] = fmaf(pi[aa].z, pj[bb].z, acc[aa][bb]);
                                acc[aa][bb] = fmaf(pi[aa].w, pj[bb].w, acc[aa][bb]);
                            }
                    }
#pragma unroll
                    for (int aa = 0; aa < 4; ++aa) {
                        float4* dst = reinterpret_cast<float4*>(T + (ti + aa * qi) * kDiagPitch + 4 * tj);
                        float4 o = *dst;
                        o.x -= acc[aa][0]; o.y -= acc[aa][1]; o.z -= acc[aa][2]; o.w -= acc[aa][3];
                        *dst = o;
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kBulkThreads) : "memory");
            }
            __threadfence_block();
            if (bt == 0) s_bulk = j + 1;
        }
    }
    __syncthreads();
    if (tid == 0 && s_bad) atomicOr(status, CRB_FLAG_BAD_PIVOT);
    if (tid == 0 && s_gave_up) atomicOr(status, CRB_FLAG_WAIT_LIMIT);

    // ---------------- phase 2: inverse by merging diagonal blocks of size s = 16, 32, 64 ----------------
    for (int s = 16; s < FB; s <<= 1) {
        const int pairs = FB / (2 * s);
        const int gthreads = kDiagThreads / pairs;                      // threads per pair
        const int pr = tid / gthreads, tg = tid % gthreads;
        const int b0 = pr * 2 * s;
        // T = L21 * Ainv   (L21 = a[b0+s.., b0..], Ainv = x[b0.., b0..])
        smem_gemm_nn<false>(a + (b0 + s) * kDiagPitch + b0, kDiagPitch, x + b0 * kDiagPitch + b0, kDiagPitch,
                            tmp + (pr * s) * kDiagTmpPitch, kDiagTmpPitch, s, tg, gthreads);
        __syncthreads();
        // X21 = -Dinv * T  (Dinv = x[b0+s.., b0+s..])
        smem_gemm_nn<true>(x + (b0 + s) * kDiagPitch + b0 + s, kDiagPitch, tmp + (pr * s) * kDiagTmpPitch, kDiagTmpPitch,
                           x + (b0 + s) * kDiagPitch + b0, kDiagPitch, s, tg, gthreads);
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < FB * FB / 4 / kDiagThreads; ++u) {
        const int e = 4 * (tid + u * kDiagThreads);
        *reinterpret_cast<float4*>(Akk + (int64_t)(e >> 7) * ld + (e & 127)) =
            *reinterpret_cast<const float4*>(x + (e >> 7) * kDiagPitch + (e & 127));
    }
}

// U = index-reversed copy of the lower-triangular X (upper triangle and diagonal; zeros below).
__global__ void k_reverse_upper(const float* __restrict__ X, int C, float* __restrict__ U) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int i = blockIdx.y;
    if (j >= C) return;
    U[(int64_t)i * C + j] = (j >= i) ? X[(int64_t)(C - 1 - i) * C + (C - 1 - j)] : 0.f;
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

size_t factor_workspace_bytes(int C) {
    if (C <= 0) return 0;
    return align256(sizeof(float) * (size_t)C * C) + 256 + align256((size_t)C);
}

// One merge of the recursion: with both halves of [lo, hi) inverted, the block below the diagonal
// becomes  -D^-1 B A^-1.  Both inverses are lower triangular: their zero halves are not multiplied.
static int merge_halves(float* A, int C, int lo, int mid, int hi, float* tmp, unsigned* status, cudaStream_t st,
                        int max_ctas) {
    const int s1 = (mid - lo) * FB, s2 = (hi - mid) * FB;
    float* B = A + (int64_t)mid * FB * C + (int64_t)lo * FB;
    const float* Ainv = A + (int64_t)lo * FB * (C + 1);
    const float* Dinv = A + (int64_t)mid * FB * (C + 1);
    int rc = gemm_tf32x3(false, GEMM_B_LOWER, s2, s1, s1, 1.0f, B, C, Ainv, C, 0.0f, tmp, s1, status, st, nullptr,
                         max_ctas);                                                                         // T = B A^-1
    if (rc != CRB_OK) return rc;
    return gemm_tf32x3(false, GEMM_A_LOWER, s2, s1, s2, -1.0f, Dinv, C, tmp, s1, 0.0f, B, C, status, st, nullptr,
                       max_ctas);                                                                           // B = -D^-1 T
}

// Inverse of the lower-triangular factor on the diagonal blocks [lo, hi), in place, by recursive
// merges (the single-panel case: everything on the caller's stream after the factorisation).
static int invert_range(float* A, int C, int lo, int hi, float* tmp, unsigned* status, cudaStream_t st) {
    if (hi - lo <= 1) return CRB_OK;
    const int mid = lo + (hi - lo) / 2;
    int rc = invert_range(A, C, lo, mid, tmp, status, st);
    if (rc != CRB_OK) return rc;
    rc = invert_range(A, C, mid, hi, tmp, status, st);
    if (rc != CRB_OK) return rc;
    return merge_halves(A, C, lo, mid, hi, tmp, status, st, 0);
}

// The merges of the same recursion tree that become possible when outer panel `panel` has been
// factored: every node whose last diagonal block lies in that panel (nodes that ended in an earlier
// panel were merged by an earlier call).  Their inputs are final: the factor's columns of a panel
// do not change after the panel's chain, and the block a merge overwrites is read by no update of
// the factorisation that can still be in flight (an update of panel q reads the rows below panel
// q + 1 from the side stream only while panel q + 1 is being factored).  Called panel by panel on the
// side stream, this leaves only the merges that need the last panel for the end.
static int invert_completed(float* A, int C, int lo, int hi, int panel, float* tmp, unsigned* status,
                            cudaStream_t st, int max_ctas) {
    if (hi - lo <= 1) return CRB_OK;
    const int last = (hi - 1) / kOuter;
    if (panel < lo / kOuter || panel > last) return CRB_OK;
    const int mid = lo + (hi - lo) / 2;
    int rc = invert_completed(A, C, lo, mid, panel, tmp, status, st, max_ctas);
    if (rc != CRB_OK) return rc;
    rc = invert_completed(A, C, mid, hi, panel, tmp, status, st, max_ctas);
    if (rc != CRB_OK) return rc;
    return last == panel ? merge_halves(A, C, lo, mid, hi, tmp, status, st, max_ctas) : (int)CRB_OK;
}

// Grid of the inverse merges that run beside the factorisation of later panels (the last panel's
// merges, with nothing left to run beside, take the whole GPU).
constexpr int kMergeCtasBeside = 64;     // measured at C = 16384: 32 CTAs 24.8 ms, 64 23.2, 96 23.4, 128 23.1
// Grid of a far update that runs beside the next panel's chain.  Measured at C = 16384 (ms per
// factorisation, 25.6-25.8 without look-ahead): 64 CTAs 27.8, 96 25.1, 128 24.0, 140 24.2, 148 24.3.
constexpr int kFactorFarCtas = 128;
// The side streams of a caller stream, and events to fork to them and join them again (common.cuh).
static std::mutex g_side_lock;
static std::map<std::pair<int, cudaStream_t>, SideContext> g_side;

SideContext* side_context(cudaStream_t main, size_t n_events) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> guard(g_side_lock);
    SideContext& ctx = g_side[std::make_pair(dev, main)];
    if (!ctx.side) {
        // same priority as the caller's stream: the side work is part of the caller's critical path
        int prio = 0;
        if (cudaStreamGetPriority(main, &prio) != cudaSuccess) prio = 0;
        if (cudaStreamCreateWithPriority(&ctx.side, cudaStreamNonBlocking, prio) != cudaSuccess) return nullptr;
        if (cudaStreamCreateWithPriority(&ctx.side2, cudaStreamNonBlocking, prio) != cudaSuccess) return nullptr;
    }
    while (ctx.events.size() < n_events) {
        cudaEvent_t e;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        ctx.events.push_back(e);
    }
    return &ctx;
}

int factor_launch(float* H, int C, float* W, int R, int64_t ldw, float percdamp, int extra_steps,
                  void* workspace, size_t workspace_bytes, unsigned* status, cudaStream_t st) {
    if (!H || !workspace || !status || C <= 0 || extra_steps < 0) return CRB_ERR_BAD_ARG;
    if (C % FB) return CRB_ERR_UNSUPPORTED;
    if (W && (R <= 0 || ldw < C)) return CRB_ERR_BAD_ARG;
    if (workspace_bytes < factor_workspace_bytes(C)) return CRB_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(H) & 15)) return CRB_ERR_BAD_ARG;
    float* A = static_cast<float*>(workspace);
    char* tail = static_cast<char*>(workspace) + align256(sizeof(float) * (size_t)C * C);
    float* damp = reinterpret_cast<float*>(tail);
    unsigned char* dead = reinterpret_cast<unsigned char*>(tail + 256);

    k_diag_prepare<<<1, 1024, 0, st>>>(H, C, percdamp, extra_steps, damp, dead);
    CRB_LAUNCHED();
    if (W) {
        k_zero_dead<<<dim3((C + 255) / 256, R < 64 ? R : 64), 256, 0, st>>>(W, R, C, ldw, dead);
        CRB_LAUNCHED();
    }
    k_reverse_copy<<<dim3((C + 255) / 256, C), 256, 0, st>>>(H, C, damp, dead, A);
    CRB_LAUNCHED();
    const int nb = C / FB;
    constexpr int kDiagSmem = kDiagSmemFloats * (int)sizeof(float);
    static PerDeviceSetup once;
    const int rc_setup = once.run([] {
        return cudaFuncSetAttribute(k_chol_diag, cudaFuncAttributeMaxDynamicSharedMemorySize, kDiagSmem) == cudaSuccess
                   ? (int)CRB_OK : (int)CRB_ERR_LAUNCH;
    });
    if (rc_setup != CRB_OK) return rc_setup;
    // Two levels of blocking: inside an outer panel of kOuter diagonal blocks the rank-128 updates
    // touch the panel's own columns only; everything right of the panel gets one update with
    // K = 8 * 128 afterwards, which is compute bound instead of re-reading the whole trailing
    // matrix once per diagonal block.
    const int n_panels = (nb + kOuter - 1) / kOuter;
    SideContext* sc = nb > kOuter ? side_context(st, 2 * (size_t)n_panels + 2) : nullptr;
    // Look-ahead over the rank-1024 updates: the next outer panel only needs its own 1024 columns,
    // so those are updated on the caller's stream and the rest of the trailing matrix on a second
    // side stream with a capped grid, beside the next panel's chain of small kernels.  Every element
    // still receives the updates panel by panel in the same order: the factor is the same bit for bit.
    const bool ahead = sc != nullptr && n_panels > 2 && g_factor_lookahead.load(std::memory_order_relaxed) != 0;
    int far_pending = -1;             // panel whose far update is in flight (events[n_panels + 1 + p] marks its end)
    // scratch of the merges (at most C^2 / 4 floats, one merge at a time): H is free once it has been copied
    float* tmp_side = H;
    for (int k0 = 0; k0 < nb; k0 += kOuter) {
        const int k1 = k0 + kOuter < nb ? k0 + kOuter : nb;
        for (int k = k0; k < k1; ++k) {
            float* Akk = A + (int64_t)k * FB * (C + 1);
            launch_chained(k_chol_diag, 1, kDiagThreads, kDiagSmem, st, Akk, (int64_t)C, status);
            CRB_LAUNCHED();
            const int rem = C - (k + 1) * FB;
            if (rem <= 0) break;
            float* panel = Akk + (int64_t)FB * C;
            int rc = gemm_tf32x3(true, 0, rem, FB, FB, 1.0f, panel, C, Akk, C, 0.0f, panel, C, status, st);   // P = A21 L^-T
            if (rc != CRB_OK) return rc;
            const int inside = (k1 - (k + 1)) * FB;         // columns of the outer panel still to factor
            rc = gemm_tf32x3(true, GEMM_LOWER_ONLY, rem, inside, FB, -1.0f, panel, C, panel, C, 1.0f, panel + FB, C,
                             status, st);                                                                   // A22[:, :inside] -= P P^T
            if (rc != CRB_OK) return rc;
        }
        if (sc) {
            // the panel's diagonal blocks and the factor entries between them are final: invert the
            // panel's part of the factor on the side stream while this stream carries on
            const int p = k0 / kOuter;
            if (cudaEventRecord(sc->events[p], st) != cudaSuccess ||
                cudaStreamWaitEvent(sc->side, sc->events[p], 0) != cudaSuccess)
                return CRB_ERR_LAUNCH;
            const int rc = invert_completed(A, C, 0, nb, p, tmp_side, status, sc->side,
                                            k1 < nb ? kMergeCtasBeside : 0);
            if (rc != CRB_OK) return rc;
        }
        const int rem = C - k1 * FB;
        if (rem <= 0) break;
        const float* P = A + (int64_t)k1 * FB * C + (int64_t)k0 * FB;     // rows below the panel, the panel's columns
        float* T = A + (int64_t)k1 * FB * (C + 1);                        // the trailing matrix
        const int kk = (k1 - k0) * FB;
        if (!ahead) {
            const int rc = gemm_tf32x3(true, GEMM_LOWER_ONLY, rem, rem, kk, -1.0f, P, C, P, C, 1.0f, T, C, status, st);
            if (rc != CRB_OK) return rc;
            continue;
        }
        const int p = k0 / kOuter;
        // the previous panel's far update wrote the columns this one is about to update
        if (far_pending >= 0 && cudaStreamWaitEvent(st, sc->events[n_panels + 1 + far_pending], 0) != cudaSuccess)
            return CRB_ERR_LAUNCH;
        far_pending = -1;
        const int near = rem < kOuter * FB ? rem : kOuter * FB;
        int rc = gemm_tf32x3(true, GEMM_LOWER_ONLY, rem, near, kk, -1.0f, P, C, P, C, 1.0f, T, C, status, st);
        if (rc != CRB_OK) return rc;
        const int far = rem - near;
        if (far <= 0) continue;
        // the panel's columns are final (events[p], recorded above for the panel-local inverse)
        if (cudaStreamWaitEvent(sc->side2, sc->events[p], 0) != cudaSuccess) return CRB_ERR_LAUNCH;
        const float* Pf = P + (int64_t)near * C;
        rc = gemm_tf32x3(true, GEMM_LOWER_ONLY, far, far, kk, -1.0f, Pf, C, Pf, C, 1.0f, T + (int64_t)near * (C + 1), C,
                         status, sc->side2, nullptr, kFactorFarCtas);
        if (rc != CRB_OK) return rc;
        if (cudaEventRecord(sc->events[n_panels + 1 + p], sc->side2) != cudaSuccess) return CRB_ERR_LAUNCH;
        far_pending = p;
    }
    if (far_pending >= 0 && cudaStreamWaitEvent(st, sc->events[n_panels + 1 + far_pending], 0) != cudaSuccess)
        return CRB_ERR_LAUNCH;
    if (sc) {
        if (cudaEventRecord(sc->events[n_panels], sc->side) != cudaSuccess ||
            cudaStreamWaitEvent(st, sc->events[n_panels], 0) != cudaSuccess)
            return CRB_ERR_LAUNCH;
    }
    if (!sc) {
        const int rc = invert_range(A, C, 0, nb, tmp_side, status, st);         // a single outer panel
        if (rc != CRB_OK) return rc;
    }
    k_reverse_upper<<<dim3((C + 255) / 256, C), 256, 0, st>>>(A, C, H);
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
