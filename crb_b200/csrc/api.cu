// extern "C" surface of libcrb_b200 (declared in include/crb_b200.h).
#include <stdio.h>

#include "common.cuh"

namespace crb {

std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_dependent_launch{1};
std::atomic<int> g_fused_selection{0};
std::atomic<int> g_trailing_lookahead{1};
std::atomic<int> g_factor_lookahead{1};

// block_step.cu
size_t block_workspace_bytes(int R);
int block_step_launch(float* W, int R, int64_t ldw, const float* U, int64_t ldu, int block,
                      int technique, int orders, float lam, float corr_damp, int metric, float* Err, int64_t ld_err,
                      float* Losses, unsigned char* codes, int64_t ld_codes, float* scales,
                      double* trace, void* workspace, size_t workspace_bytes, cudaStream_t st, bool reset_tickets = true);
int binarize_group_launch(const float* W, int R, int64_t ldw, const unsigned char* mask, int64_t ldm,
                          int order, int technique, float lam, float corr_damp, float* Q, int64_t ldq,
                          cudaStream_t st);
// dequant.cu
int dequantize_launch(float* W, int R, int C, int64_t ldw, int technique, const unsigned char* b1,
                      const unsigned char* lm, const unsigned char* salcol, const unsigned char* b2,
                      const long long* b2_off, const int* b2_pitch, const float* scales, cudaStream_t st);
// hessian.cu
size_t hessian_workspace_bytes(int C, int64_t T, int dtype);
int hessian_accumulate_launch(const void* X, int dtype, int64_t T, int C, int64_t ldx, float* S,
                              void* workspace, size_t workspace_bytes, cudaStream_t st);
int hessian_finalize_launch(float* S, int C, float scale, cudaStream_t st);
long long hessian_packed_floats(int C);
int hessian_pack_launch(float* S, int C, float* packed, int unpack, cudaStream_t st);
// factor.cu
size_t factor_workspace_bytes(int C);
int factor_launch(float* H, int C, float* W, int R, int64_t ldw, float percdamp, int extra_steps,
                  void* workspace, size_t workspace_bytes, unsigned* status, cudaStream_t st);

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace crb

using namespace crb;

extern "C" {

int crb_version(void) { return 2; }

const char* crb_arch(void) { return "sm_100a"; }

const char* crb_status_string(int status) {
    switch (status) {
        case CRB_OK: return "ok";
        case CRB_ERR_BAD_ARG: return "bad argument";
        case CRB_ERR_WORKSPACE: return "workspace too small";
        case CRB_ERR_LAUNCH: return "CUDA launch or API call failed";
        case CRB_ERR_UNSUPPORTED: return "unsupported shape or option";
        case CRB_ERR_STATIC_LIMIT: return "row count exceeds the built-in scratch of crb_block_step_static";
        default: return status > 0 ? "device status flags" : "unknown error";
    }
}

int crb_set_dependent_launch(int enable) {
    return g_dependent_launch.exchange(enable ? 1 : 0);
}

int crb_set_factor_lookahead(int enable) {
    return g_factor_lookahead.exchange(enable ? 1 : 0);
}

int crb_set_trailing_lookahead(int mode) {
    return g_trailing_lookahead.exchange(mode < 0 ? 0 : mode > 2 ? 2 : mode);
}

int crb_set_fused_selection(int enable) {
    return g_fused_selection.exchange(enable ? 1 : 0);
}

unsigned long long crb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t crb_hessian_workspace_bytes(int C, int64_t T, int dtype) { return hessian_workspace_bytes(C, T, dtype); }

int crb_hessian_accumulate(const void* X, int dtype, int64_t T, int C, int64_t ldx, float* S,
                           void* workspace, size_t workspace_bytes, void* stream) {
    return hessian_accumulate_launch(X, dtype, T, C, ldx, S, workspace, workspace_bytes,
                                     static_cast<cudaStream_t>(stream));
}

int crb_hessian_finalize(float* S, int C, float scale, void* stream) {
    return hessian_finalize_launch(S, C, scale, static_cast<cudaStream_t>(stream));
}

size_t crb_hessian_packed_floats(int C) { return (size_t)hessian_packed_floats(C); }

int crb_hessian_pack(const float* S, int C, float* packed, void* stream) {
    return hessian_pack_launch(const_cast<float*>(S), C, packed, 0, static_cast<cudaStream_t>(stream));
}

int crb_hessian_unpack(const float* packed, int C, float* S, void* stream) {
    return hessian_pack_launch(S, C, const_cast<float*>(packed), 1, static_cast<cudaStream_t>(stream));
}

size_t crb_factor_workspace_bytes(int C) { return factor_workspace_bytes(C); }

int crb_hinv_upper_factor(float* H, int C, float* W, int R, int64_t ldw, float percdamp,
                          int extra_damp_steps, void* workspace, size_t workspace_bytes,
                          unsigned* status, void* stream) {
    return factor_launch(H, C, W, R, ldw, percdamp, extra_damp_steps, workspace, workspace_bytes, status,
                         static_cast<cudaStream_t>(stream));
}

size_t crb_block_workspace_bytes(int R) { return R > 0 ? block_workspace_bytes(R) : 0; }

int crb_block_step(float* W, int R, int64_t ldw, const float* U, int64_t ldu, int block,
                   int technique, int orders, float lam, float corr_damp, int metric, float* Err, float* Losses,
                   uint8_t* codes, float* scales, double* trace, void* workspace,
                   size_t workspace_bytes, void* stream) {
    // `codes` is [R, 128] for a single block: offset the base so that column (block*128 + j)
    // of a virtual [R, ldw]-wide buffer lands on codes[r, j].
    uint8_t* codes_base = codes ? codes - (int64_t)block * kBlock : nullptr;
    return block_step_launch(W, R, ldw, U, ldu, block, technique, orders, lam, corr_damp, metric, Err, kBlock, Losses,
                             codes_base, kBlock, scales, trace, workspace, workspace_bytes,
                             static_cast<cudaStream_t>(stream));
}

int crb_binarize_group(const float* W, int R, int64_t ldw, const uint8_t* mask, int64_t ldm, int order,
                       int technique, float lam, float corr_damp, float* Q, int64_t ldq, void* stream) {
    return binarize_group_launch(W, R, ldw, mask, ldm, order, technique, lam, corr_damp, Q, ldq,
                                 static_cast<cudaStream_t>(stream));
}

static int trailing_update_impl(float* W, int R, int C, int64_t ldw, const float* Err, const float* U,
                                int64_t ldu, int block, unsigned* status, cudaStream_t st) {
    if (!W || !Err || !U || R <= 0 || C <= 0 || (C % kBlock) || block < 0) return CRB_ERR_BAD_ARG;
    const int ed = (block + 1) * kBlock;
    if (ed > C) return CRB_ERR_BAD_ARG;
    if (ed == C) return CRB_OK;
    return gemm_tf32x3(false, 0, R, C - ed, kBlock, -1.0f, Err, kBlock, U + (int64_t)block * kBlock * ldu + ed,
                       ldu, 1.0f, W + ed, ldw, status, st);
}

int crb_trailing_update(float* W, int R, int C, int64_t ldw, const float* Err, const float* U,
                        int64_t ldu, int block, void* stream) {
    return trailing_update_impl(W, R, C, ldw, Err, U, ldu, block, nullptr, static_cast<cudaStream_t>(stream));
}

int crb_gemm_f32(int b_is_nk, int shape, int M, int N, int K, float alpha, const float* A, int64_t lda,
                 const float* B, int64_t ldb, float beta, float* C, int64_t ldc, unsigned* status, void* stream) {
    return gemm_tf32x3(b_is_nk != 0, shape, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, status,
                       static_cast<cudaStream_t>(stream));
}

// Blocks per group of the block loop.  Inside a group a block's error is propagated to the group's
// remaining columns right away (K = 128); the columns right of the group receive the group's
// errors in one product with K = kGroup * 128 once its last block is done.  The sums are the ones
// of bigptq.py:264, associated differently; the trailing part of W is read and written once per
// group instead of once per block.
constexpr int kGroup = 8;

static_assert(CRB_GEMM_LOWER_ONLY == GEMM_LOWER_ONLY && CRB_GEMM_B_LOWER == GEMM_B_LOWER &&
              CRB_GEMM_A_LOWER == GEMM_A_LOWER, "shape flags of the header and of the kernel");

size_t crb_linear_workspace_bytes(int R) {
    if (R <= 0) return 0;
    // block-step scratch + the errors of two groups of blocks (the current one, and the previous one
    // while its trailing update may still be running beside the current group)
    return align256(block_workspace_bytes(R)) + 2 * align256(sizeof(float) * (size_t)R * kBlock * kGroup);
}

// Grid of the far part of a trailing update when it runs beside the next group's block steps: the
// rest of the SMs stays with the block steps and their in-group products.
constexpr int kFarCtas = 64;      // measured at 4096 x 16384: 40 -> 20.8 ms per loop, 64 / 96 -> 18.6 ms (19.8 without look-ahead)

int crb_quantize_linear(float* W, int R, int C, int64_t ldw, const float* U, int64_t ldu,
                        int technique, int orders, float lam, float corr_damp, int metric, float* Losses,
                        uint8_t* codes, float* scales, double* trace, void* workspace,
                        size_t workspace_bytes, void* stream) {
    if (!W || !U || !Losses || !workspace || R <= 0 || C <= 0) return CRB_ERR_BAD_ARG;
    if (C % kBlock) return CRB_ERR_UNSUPPORTED;
    if (workspace_bytes < crb_linear_workspace_bytes(R)) return CRB_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t bws = align256(block_workspace_bytes(R));
    const size_t group_bytes = align256(sizeof(float) * (size_t)R * kBlock * kGroup);
    const int64_t ld_err = (int64_t)kGroup * kBlock;
    unsigned* status = static_cast<unsigned*>(workspace);
    if (cudaMemsetAsync(workspace, 0, 64, st) != cudaSuccess) return CRB_ERR_LAUNCH;   // status word
    const int nblk = C / kBlock, grp = kGroup;
    const int ngroups = (nblk + grp - 1) / grp;
    // Look-ahead over the trailing updates.  After a group of 8 blocks every later column needs
    // W -= Err_group U[group rows, column], but the next group only needs its own 1024 columns.
    // Those are updated on the caller's stream; the rest (a large product at the GEMM's full rate)
    // runs on a side stream with a capped grid beside the next group's block steps, which are
    // chains of short kernels.  Every element still receives its updates group by group in the
    // same order and from the same products, so the result is the same bit for bit.  It pays for
    // wide, short weights (the trailing products are a quarter of the loop at 4096 x 16384); the
    // block steps of tall weights need all SMs themselves.
    const int mode = g_trailing_lookahead.load(std::memory_order_relaxed);
    const bool ahead = ngroups > 2 && (mode == 2 || (mode == 1 && C >= 8192 && R <= 8192));
    SideContext* sc = ahead ? side_context(st, (size_t)ngroups + 1) : nullptr;
    if (ahead && !sc) return CRB_ERR_LAUNCH;
    int far_pending = -1;           // group whose far update is in flight on the side stream (events[g] marks its end)
    for (int b = 0; b < nblk; ++b) {
        const int g = b / grp, g0 = g * grp, g1 = g0 + grp < nblk ? g0 + grp : nblk;
        float* ErrG = reinterpret_cast<float*>(static_cast<char*>(workspace) + bws + (size_t)(ahead ? g & 1 : 0) * group_bytes);
        float* Err = ErrG + (size_t)(b - g0) * kBlock;
        int rc = block_step_launch(W, R, ldw, U, ldu, b, technique, orders, lam, corr_damp, metric, Err, ld_err, Losses, codes,
                                   C, scales ? scales + (size_t)b * R * 8 : nullptr,
                                   trace ? trace + (size_t)b * CRB_TRACE_DOUBLES : nullptr, workspace, bws, st, b == 0);
        if (rc != CRB_OK) return rc;
        const int ed = (b + 1) * kBlock;
        rc = gemm_tf32x3(false, 0, R, g1 * kBlock - ed, kBlock, -1.0f, Err, ld_err,
                         U + (int64_t)b * kBlock * ldu + ed, ldu, 1.0f, W + ed, ldw, status, st);
        if (rc != CRB_OK) return rc;
        if (b != g1 - 1 || g1 >= nblk) continue;
        const int gd = g1 * kBlock, kk = (g1 - g0) * kBlock;
        const float* Ug = U + (int64_t)g0 * kBlock * ldu;
        if (!ahead) {
            rc = gemm_tf32x3(false, 0, R, C - gd, kk, -1.0f, ErrG, ld_err, Ug + gd, ldu, 1.0f, W + gd, ldw, status, st);
            if (rc != CRB_OK) return rc;
            continue;
        }
        // the previous group's far update wrote the columns this one is about to update (and has
        // read the error buffer the next group will overwrite)
        if (far_pending >= 0 && cudaStreamWaitEvent(st, sc->events[far_pending], 0) != cudaSuccess) return CRB_ERR_LAUNCH;
        far_pending = -1;
        const int near = C - gd < grp * kBlock ? C - gd : grp * kBlock;
        rc = gemm_tf32x3(false, 0, R, near, kk, -1.0f, ErrG, ld_err, Ug + gd, ldu, 1.0f, W + gd, ldw, status, st);
        if (rc != CRB_OK) return rc;
        const int far = C - gd - near;
        if (far <= 0) continue;
        // fork: the side stream starts once this group's errors are complete (they are: the near
        // update above is ordered behind them on this stream)
        if (cudaEventRecord(sc->events[ngroups], st) != cudaSuccess ||
            cudaStreamWaitEvent(sc->side, sc->events[ngroups], 0) != cudaSuccess)
            return CRB_ERR_LAUNCH;
        rc = gemm_tf32x3(false, 0, R, far, kk, -1.0f, ErrG, ld_err, Ug + gd + near, ldu, 1.0f, W + gd + near, ldw,
                         status, sc->side, nullptr, kFarCtas);
        if (rc != CRB_OK) return rc;
        if (cudaEventRecord(sc->events[g], sc->side) != cudaSuccess) return CRB_ERR_LAUNCH;
        far_pending = g;
    }
    if (far_pending >= 0 && cudaStreamWaitEvent(st, sc->events[far_pending], 0) != cudaSuccess) return CRB_ERR_LAUNCH;
    return CRB_OK;
}

int crb_dequantize(float* W, int R, int C, int64_t ldw, int technique, const uint8_t* b1, const uint8_t* lm,
                   const uint8_t* salcol, const uint8_t* b2, const int64_t* b2_off, const int32_t* b2_pitch,
                   const float* scales, void* stream) {
    return dequantize_launch(W, R, C, ldw, technique, b1, lm, salcol, b2,
                             reinterpret_cast<const long long*>(b2_off), b2_pitch, scales,
                             static_cast<cudaStream_t>(stream));
}

int crb_selftest_wait_limit(void* scratch, size_t scratch_bytes, unsigned limit_us, unsigned* status,
                            void* stream) {
    constexpr int M = 128, N = 256, K = 32;
    if (!scratch || !status || scratch_bytes < (size_t)256 * 1024 || limit_us == 0) return CRB_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(scratch) & 255) return CRB_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(scratch, 0, (size_t)256 * 1024, st) != cudaSuccess) return CRB_ERR_LAUNCH;
    float* A = static_cast<float*>(scratch);
    float* B = A + M * K;
    float* C = B + N * K;
    GemmSelfTest t;
    t.wait_ns = (unsigned long long)limit_us * 1000ull;
    t.withhold_loads = 1;
    return gemm_tf32x3(true, 0, M, N, K, 1.0f, A, K, B, K, 0.0f, C, N, status, st, &t);
}

int crb_read_status(const void* workspace, void* stream) {
    if (!workspace) return CRB_ERR_BAD_ARG;
    unsigned flags = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&flags, workspace, sizeof(flags), cudaMemcpyDeviceToHost, st) != cudaSuccess)
        return CRB_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return CRB_ERR_LAUNCH;
    return (int)(flags & 0x7fffffffu);
}

}  // extern "C"
