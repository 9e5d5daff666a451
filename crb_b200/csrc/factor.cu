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
// Blocked with 128-wide panels.  Per panel: one CTA factors the 128x128 diagonal block in
// shared memory and inverts it; the panel below is multiplied by that inverse and the trailing
// matrix gets a rank-128 update, both through the split-TF32 tensor-core GEMM (gemm_tc.cu).  The triangular inverse
// merges neighbouring diagonal blocks recursively: [[A,0],[B,D]]^-1 = [[A^-1,0],[-D^-1 B A^-1, D^-1]].
// A non-positive pivot sets CRB_FLAG_BAD_PIVOT (the host re-damps and calls again, like the
// retry loop at bigptq.py:115-123) and is replaced by 1 so that nothing non-finite spreads.
#include "common.cuh"

namespace crb {

int gemm_tf32x3(bool b_is_nk, bool lower_only, int M, int N, int K, float alpha, const float* A, int64_t lda,
                const float* B, int64_t ldb, float beta, float* C, int64_t ldc, unsigned* status,
                cudaStream_t st);

constexpr int FB = 128;    // panel width

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

// Factor one 128x128 diagonal block (lower Cholesky, left-looking) and overwrite it with the
// inverse of its factor (zeros above the diagonal).  512 threads: four lanes share a row (or a
// column of the inverse) and split every dot product four ways, so that the serial chain per
// column is a quarter of the row length plus two shuffles.
constexpr int kDiagThreads = 4 * FB;
constexpr int kDiagPitch = FB + 4;

__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

__global__ void __launch_bounds__(kDiagThreads)
k_chol_diag(float* __restrict__ Akk, int64_t ld, unsigned* status) {
    // row pitch 132 floats: the four lanes of a row and the eight rows of a warp hit 32 distinct banks
    extern __shared__ float s_diag[];
    float (*a)[kDiagPitch] = reinterpret_cast<float (*)[kDiagPitch]>(s_diag);
    float (*x)[kDiagPitch] = reinterpret_cast<float (*)[kDiagPitch]>(s_diag + FB * kDiagPitch);
    const int tid = threadIdx.x;
    const int i = tid >> 2, s = tid & 3;               // row (phase 1) / column (phase 2), quarter
    for (int e = tid; e < FB * FB; e += kDiagThreads) a[e >> 7][e & 127] = Akk[(int64_t)(e >> 7) * ld + (e & 127)];
    __syncthreads();
    bool bad = false;
    for (int k = 0; k < FB; ++k) {
        // column k: acc = a[i][k] - sum_{j<k} a[i][j] * a[k][j]   for rows i >= k
        float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
        if (i >= k) {
            int j = s;
            for (; j + 12 < k; j += 16) {          // four independent chains keep the loads in flight
                p0 = fmaf(a[i][j], a[k][j], p0);
                p1 = fmaf(a[i][j + 4], a[k][j + 4], p1);
                p2 = fmaf(a[i][j + 8], a[k][j + 8], p2);
                p3 = fmaf(a[i][j + 12], a[k][j + 12], p3);
            }
            for (; j < k; j += 4) p0 = fmaf(a[i][j], a[k][j], p0);
        }
        const float acc = a[i][k] - quad_sum((p0 + p1) + (p2 + p3));
        if (i == k && s == 0) {
            float piv = acc;
            if (!(piv > 0.f) || !isfinite(piv)) { bad = true; piv = 1.f; }
            a[k][k] = sqrtf(piv);
        }
        __syncthreads();
        if (i > k && s == 0) a[i][k] = __fdiv_rn(acc, a[k][k]);
        __syncthreads();
    }
    if (bad) atomicOr(status, CRB_FLAG_BAD_PIVOT);
    // inverse of the lower factor by forward substitution, column j = tid / 4:
    //   x[r][j] = (delta_rj - sum_{m=j}^{r-1} a[r][m] x[m][j]) / a[r][r]
    // rows are produced in order; the four lanes of a column split the sum over m.
    const int j = i;
    for (int r = 0; r < FB; ++r) {
        float p = 0.f, pb = 0.f;
        if (r > j) {
            int m = j + s;
            for (; m + 4 < r; m += 8) {
                p = fmaf(a[r][m], x[m][j], p);
                pb = fmaf(a[r][m + 4], x[m + 4][j], pb);
            }
            if (m < r) p = fmaf(a[r][m], x[m][j], p);
        }
        p = quad_sum(p + pb);
        if (s == 0) x[r][j] = (r < j) ? 0.f : ((r == j) ? __fdiv_rn(1.f, a[r][r]) : __fdiv_rn(-p, a[r][r]));
        __syncwarp();
    }
    __syncthreads();
    for (int e = tid; e < FB * FB; e += kDiagThreads) Akk[(int64_t)(e >> 7) * ld + (e & 127)] = x[e >> 7][e & 127];
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

static int invert_range(float* A, int C, int lo, int hi, float* tmp, unsigned* status, cudaStream_t st) {
    if (hi - lo <= 1) return CRB_OK;
    const int mid = lo + (hi - lo) / 2;
    int rc = invert_range(A, C, lo, mid, tmp, status, st);
    if (rc != CRB_OK) return rc;
    rc = invert_range(A, C, mid, hi, tmp, status, st);
    if (rc != CRB_OK) return rc;
    const int s1 = (mid - lo) * FB, s2 = (hi - mid) * FB;
    float* B = A + (int64_t)mid * FB * C + (int64_t)lo * FB;
    const float* Ainv = A + (int64_t)lo * FB * (C + 1);
    const float* Dinv = A + (int64_t)mid * FB * (C + 1);
    rc = gemm_tf32x3(false, false, s2, s1, s1, 1.0f, B, C, Ainv, C, 0.0f, tmp, s1, status, st);      // T = B A^-1
    if (rc != CRB_OK) return rc;
    return gemm_tf32x3(false, false, s2, s1, s2, -1.0f, Dinv, C, tmp, s1, 0.0f, B, C, status, st);   // B = -D^-1 T
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
    constexpr int kDiagSmem = 2 * FB * kDiagPitch * (int)sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_chol_diag, cudaFuncAttributeMaxDynamicSharedMemorySize, kDiagSmem) != cudaSuccess)
            return CRB_ERR_LAUNCH;
        attr_set = true;
    }
    for (int k = 0; k < nb; ++k) {
        float* Akk = A + (int64_t)k * FB * (C + 1);
        k_chol_diag<<<1, kDiagThreads, kDiagSmem, st>>>(Akk, C, status);
        CRB_LAUNCHED();
        const int rem = C - (k + 1) * FB;
        if (rem <= 0) break;
        float* panel = Akk + (int64_t)FB * C;
        int rc = gemm_tf32x3(true, false, rem, FB, FB, 1.0f, panel, C, Akk, C, 0.0f, panel, C, status, st);   // P = A21 L^-T
        if (rc != CRB_OK) return rc;
        rc = gemm_tf32x3(true, true, rem, rem, FB, -1.0f, panel, C, panel, C, 1.0f, panel + FB, C, status, st);  // A22 -= P P^T
        if (rc != CRB_OK) return rc;
    }
    int rc = invert_range(A, C, 0, nb, H, status, st);          // H is free to serve as scratch now
    if (rc != CRB_OK) return rc;
    k_reverse_upper<<<dim3((C + 255) / 256, C), 256, 0, st>>>(A, C, H);
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
