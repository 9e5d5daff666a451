/*
 * crb_b200 -- C ABI of the B200 (sm_100a) implementation of the CRB / BiLLM
 * calibration-time binarization path.
 *
 * Conventions
 *   - every pointer named *_dev / documented "device" is a CUDA device pointer
 *     on the current device; `stream` is a cudaStream_t passed as void*;
 *   - matrices are row-major float32 unless a dtype argument says otherwise;
 *   - all calls are asynchronous on `stream`, take caller-allocated workspace
 *     and return a crbStatus (0 = ok, <0 = bad arguments / launch failure);
 *     data-dependent conditions (non-finite input, failed pivot) are written
 *     to a device status word that crb_read_status() copies back;
 *   - the block width is fixed at 128 columns (the reference's --blocksize 128)
 *     and the column count must be a multiple of 128.
 *
 * The reference has no FFI on this path; each entry point names the Python
 * code of the reference that it replaces (paths inside the reference project).
 */
#ifndef CRB_B200_H
#define CRB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CRB_BLOCK 128          /* columns per block step                       */
#define CRB_SALIENT_LIMIT 50   /* utils/structure.py:16 (up_lim)               */
#define CRB_N_SPLITS 81        /* utils/autosearch.py:65                       */
#define CRB_TRACE_DOUBLES 320  /* doubles per block in the search trace        */

typedef enum {
    CRB_OK = 0,
    CRB_ERR_BAD_ARG = -1,
    CRB_ERR_WORKSPACE = -2,    /* workspace too small                          */
    CRB_ERR_LAUNCH = -3,       /* a CUDA launch / API call failed              */
    CRB_ERR_UNSUPPORTED = -4,  /* shape or option outside what is implemented  */
    CRB_ERR_STATIC_LIMIT = -5  /* more rows than the built-in scratch can serve */
} crbStatus;

/* Binarization.quantize dispatch (binary.py:2875-2890): braq, crbog, crb (v7) and the three flag
 * variants of v7: no sign refinement (skip_refinement), symmetric correlation damping. */
typedef enum {
    CRB_TECH_BRAQ = 0,
    CRB_TECH_CRBOG = 1,
    CRB_TECH_CRB = 2,
    CRB_TECH_CRB_NOREFINE = 3,
    CRB_TECH_CRB_SYMDAMP = 4,
    CRB_TECH_CRB_SYMDAMP_NOREFINE = 5
} crbTechnique;
/* `orders` arguments: expansions of the (low, mid, salient) groups as decimal digits, each 1 or 2;
 * 112 is the reference's default orders=(1, 1, 2) (bigptq.py:56, :246-247). */
#define CRB_ORDERS_DEFAULT 112
typedef enum { CRB_METRIC_HESSIAN = 0, CRB_METRIC_MAGNITUDE = 1 } crbMetric;
typedef enum { CRB_F32 = 0, CRB_F16 = 1, CRB_BF16 = 2 } crbDtype;

/* bits of the device status word (crb_read_status) */
#define CRB_FLAG_NONFINITE   1u   /* a non-finite metric / error was seen       */
#define CRB_FLAG_BAD_PIVOT   2u   /* factorisation met a non-positive pivot     */
#define CRB_FLAG_WAIT_LIMIT  4u   /* a bounded wait in a kernel ran out         */

/* Layout of one block's search trace (CRB_TRACE_DOUBLES doubles):
 *   [0] salient column count i*        [1] split index k*      [2] split value p*
 *   [3] relative gap to the runner-up salient count            [4] same for the split
 *   [5] mean squared error of the salient group (constant term of the split search)
 *   [6..55]   the 50 highest-score columns, best first
 *   [56..104] mean squared error of salient candidates i = 1..49
 *   [105..185] mean squared error of split candidates k = 0..80
 *   [186..266] the 81 split candidates (quantiles 0.10 .. 0.90 of the non-salient metric)
 *   [267..316] the column scores (sums of the metric over the rows) of the 50 columns in [6..55]
 */

int crb_version(void);
/* compiled architecture string, e.g. "sm_100a" */
const char *crb_arch(void);
const char *crb_status_string(int status);

/* ---- (1) Hessian accumulation --------------------------------------------------
 * Replaces BRAGPTQ.add_batch (bigptq.py:37-54).  S += X^T X for X [T, C] (row
 * major, leading dimension ldx elements) of dtype f16/bf16/f32, accumulated in
 * float32.  S is the UNSCALED sum; crb_hessian_finalize applies 2/N once, which
 * equals the reference's running rescale (bigptq.py:50-53) up to rounding.     */
size_t crb_hessian_workspace_bytes(int C, int64_t T, int dtype);
int crb_hessian_accumulate(const void *X_dev, int dtype, int64_t T, int C, int64_t ldx,
                           float *S_dev, void *workspace_dev, size_t workspace_bytes,
                           void *stream);
/* H = scale * S, both triangles written (S holds the upper-triangle tiles). */
int crb_hessian_finalize(float *S_dev, int C, float scale, void *stream);

/* The part of S that crb_hessian_accumulate maintains (the 256 x 256 tiles on and above the
 * diagonal) as one contiguous buffer of crb_hessian_packed_floats(C) floats and back: what a sum of
 * partial Hessians over several GPUs has to move (about half of C * C).  No counterpart in the
 * single-device reference; the sum itself stands for the accumulation over all sequences in
 * bigptq.py:50-53.  The packed buffer must be 16-byte aligned.                                  */
size_t crb_hessian_packed_floats(int C);
int crb_hessian_pack(const float *S_dev, int C, float *packed_dev, void *stream);
int crb_hessian_unpack(const float *packed_dev, int C, float *S_dev, void *stream);

/* ---- (2) damping + inverse factor ----------------------------------------------
 * Replaces bigptq.py:101-129: dead columns (diag == 0 -> H[d,d] = 1, W[:,d] = 0),
 * H += percdamp * mean(diag) * I, then U = chol(inv(H), upper) written over H.
 * `extra_damp_steps` >= 0 adds that many times 1e-3 * mean(diag) first (the
 * reference's retry, bigptq.py:115-123, driven by the host after it reads
 * CRB_FLAG_BAD_PIVOT).  W may be NULL.                                          */
size_t crb_factor_workspace_bytes(int C);
int crb_hinv_upper_factor(float *H_dev, int C, float *W_dev, int R, int64_t ldw, float percdamp,
                          int extra_damp_steps, void *workspace_dev, size_t workspace_bytes,
                          unsigned *status_dev, void *stream);

/* ---- (3) block step -------------------------------------------------------------
 * Replaces one iteration of the block loop, bigptq.py:142-263 with
 * utils/structure.py:8-20, utils/autosearch.py:28-83, utils/mask.py:7-18 and the
 * binarizers binary.py:18-39 (braq), :577-687 (crbog), :1544-1638 (crb).
 *   W     [R, ldw]  in: current weights; out: columns of the block replaced by Q
 *   U     [C, ldu]  upper factor; only diag of the block is read
 *   Err   [R, 128]  out: (w - q) / d
 *   Losses[R]       in/out: += sum_j (w - q)^2 / d^2 / 2
 *   codes [R, 128]  optional (NULL): bits 0-1 B1+1, bits 2-3 B2+1, bits 4-5 group
 *   scales[R, 8]    optional (NULL): per-row scales, see the Python docs; only with orders 112
 *   trace [320]     optional (NULL): doubles, layout above                       */
size_t crb_block_workspace_bytes(int R);
int crb_block_step(float *W_dev, int R, int64_t ldw, const float *U_dev, int64_t ldu, int block,
                   int technique, int orders, float lam, float corr_damp, int metric, float *Err_dev,
                   float *Losses_dev, uint8_t *codes_dev, float *scales_dev, double *trace_dev,
                   void *workspace_dev, size_t workspace_bytes, void *stream);

/* ---- block step without a workspace ----------------------------------------------------
 * No counterpart in the reference: an addition for callers that cannot allocate device
 * memory when they need a block step (an operator hook inside a framework that owns the
 * whole GPU through its own memory pool; a latency-critical loop that cannot take the
 * device-wide synchronisation of cudaMalloc / cudaFree).  Same arithmetic, arguments and
 * outputs as crb_block_step, but the scratch memory is an array inside the library image
 * (23 MiB on every GPU that loads the library) instead of a caller workspace, and the call
 * performs no allocation of any kind.
 *   - R <= CRB_STATIC_MAX_ROWS, otherwise CRB_ERR_STATIC_LIMIT and nothing is launched;
 *   - flags_out (optional, device): receives this call's status flags (CRB_FLAG_*);
 *   - all calls on one device share the array: calls that overlap on the GPU race, so order
 *     them on one stream (or with events);
 *   - the first call on each device looks up the array's device address, and where the CUDA
 *     runtime loads modules lazily that look-up is also what loads the library's device code
 *     (the array included) onto the GPU: "no allocation" holds from the second call on.  Make
 *     that first call before starting any stream capture.                                   */
#define CRB_STATIC_MAX_ROWS 16384
int crb_block_step_static_max_rows(void);
int crb_block_step_static(float *W_dev, int R, int64_t ldw, const float *U_dev, int64_t ldu, int block,
                          int technique, int orders, float lam, float corr_damp, int metric, float *Err_dev,
                          float *Losses_dev, uint8_t *codes_dev, float *scales_dev, double *trace_dev,
                          unsigned *flags_out_dev, void *stream);

/* ---- group binarizer ---------------------------------------------------------------
 * Replaces Binarization.quantize (binary.py:2868-2884) for braq / crbog / crb on one
 * [R, 128] block: Q = binarizer(W on mask, order in {1, 2}), zero outside the mask.
 * mask [R, ldm] bytes (non-zero = member).  The block step applies the same device
 * code to its three groups; this entry point serves callers that bring their own mask. */
int crb_binarize_group(const float *W_dev, int R, int64_t ldw, const uint8_t *mask_dev, int64_t ldm,
                       int order, int technique, float lam, float corr_damp, float *Q_dev,
                       int64_t ldq, void *stream);

/* ---- (4) trailing update -------------------------------------------------------
 * Replaces bigptq.py:264:  W[:, (block+1)*128:] -= Err @ U[block rows, (block+1)*128:]. */
int crb_trailing_update(float *W_dev, int R, int C, int64_t ldw, const float *Err_dev,
                        const float *U_dev, int64_t ldu, int block, void *stream);

/* ---- float32 GEMM building block ------------------------------------------------------
 * C[M,N] = alpha * A[M,K] * op(B) + beta * C, all float32 row-major, computed on the tensor
 * cores with a hi/lo TF32 split of both operands (three products per term, float32
 * accumulation), which keeps float32-level accuracy; this is what stands in for the
 * reference's TF32-disabled torch matmuls (bigptq.py:11-12, :264 and the factorisation).
 * b_is_nk != 0: B is [N, K]; else B is [K, N].  `shape` is a set of CRB_GEMM_* flags:
 * LOWER_ONLY writes only the 128 x 128 blocks of C on or below its diagonal; B_LOWER promises
 * a lower-triangular [K, N] operand B (needs b_is_nk == 0, N <= K) and A_LOWER a
 * lower-triangular A (M <= K): the zero part of such an operand is not multiplied.
 * K % 16 == 0, N % 32 == 0, leading dimensions % 4 == 0; status (device, may be NULL).   */
#define CRB_GEMM_LOWER_ONLY 1
#define CRB_GEMM_B_LOWER 2
#define CRB_GEMM_A_LOWER 4
int crb_gemm_f32(int b_is_nk, int shape, int M, int N, int K, float alpha, const float *A_dev,
                 int64_t lda, const float *B_dev, int64_t ldb, float beta, float *C_dev, int64_t ldc,
                 unsigned *status_dev, void *stream);

/* ---- packed result -> float32 weights ---------------------------------------------
 * Rebuilds W [R, C] from the packed form of a binarized linear (the reference only keeps the
 * de-quantized weights, bigptq.py:276-280; its --save is commented out, run.py:1033-1039).
 * All planes are LSB-first bit planes over the columns of a row:
 *   b1 [R, C/8]      first sign (+1 if set)        lm [R, C/8]   mid group (else low)
 *   salcol [C]       position of the column in its block's salient set, 255 = not salient
 *   b2               per block b an [R, b2_pitch[b]] plane at byte offset b2_off[b]: second sign
 *                    of the k-th salient column
 *   scales [C/128, R, 8]  as written by crb_block_step / crb_quantize_linear
 * Elements with a sign of 0 or outside every group are not representable and must be patched
 * by the caller (crb_b200/packed.py lists them with their values).                      */
int crb_dequantize(float *W_dev, int R, int C, int64_t ldw, int technique, const uint8_t *b1_dev,
                   const uint8_t *lm_dev, const uint8_t *salcol_dev, const uint8_t *b2_dev,
                   const int64_t *b2_off_dev, const int32_t *b2_pitch_dev, const float *scales_dev,
                   void *stream);

/* ---- whole linear ----------------------------------------------------------------
 * The block loop of BRAGPTQ.fasterquant (bigptq.py:131-264) for all C/128 blocks:
 * block step + trailing update, no host synchronisation.  The updates are grouped: a block's
 * error reaches the rest of its group of 8 blocks at once and the columns right of the group
 * in one product per group (same sums as bigptq.py:264, associated differently).  Buffers as above;
 * codes [R, C], scales [C/128, R, 8], trace [C/128, 320] are optional.
 * Workspace: crb_linear_workspace_bytes(R).                                       */
size_t crb_linear_workspace_bytes(int R);
int crb_quantize_linear(float *W_dev, int R, int C, int64_t ldw, const float *U_dev, int64_t ldu,
                        int technique, int orders, float lam, float corr_damp, int metric,
                        float *Losses_dev, uint8_t *codes_dev, float *scales_dev,
                        double *trace_dev, void *workspace_dev, size_t workspace_bytes,
                        void *stream);

/* Copies the status word at the start of a block/linear workspace to the host
 * (synchronises `stream`).  Returns the flags (>= 0) or a negative crbStatus.    */
int crb_read_status(const void *workspace_dev, void *stream);

/* Number of kernels this library has launched since load (for launch accounting). */
unsigned long long crb_launch_count(void);

/* Programmatic dependent launch for the chains of short kernels (block step, factorisation,
 * trailing updates): a kernel may be scheduled while its predecessor in the stream still runs and
 * waits on the device for its completion before it touches global memory.  Results are the same
 * with and without; the switch exists to measure the effect.  Returns the previous setting
 * (default 1 = on).  No counterpart in the reference (eager PyTorch launches).               */
int crb_set_dependent_launch(int enable);

/* The quantile selection of the block step as ONE cooperative kernel whose CTAs (one per SM at
 * most, all resident) meet at three bounded grid barriers, instead of three stream-ordered
 * kernels.  Same results; off by default: a cooperative launch needs all its CTAs resident at
 * once, so it waits for the whole GPU whenever other streams are busy, which costs more in the
 * layer loop (six linears on six streams) than the two kernel boundaries it saves.  Returns the
 * previous setting.  No counterpart in the reference.                                        */
int crb_set_fused_selection(int enable);

/* Look-ahead over the grouped trailing updates of crb_quantize_linear: after a group of 8 blocks
 * only the next group's columns are updated on the caller's stream; the rest of the update runs
 * on a side stream (capped grid) beside the next group's block steps.  Bit-identical results.
 * mode 0: off; 1 (default): for wide, short weights (C >= 8192 and R <= 8192), where the trailing
 * products are a quarter of the loop; 2: whenever there are more than two groups.  Returns the
 * previous mode.  No counterpart in the reference (bigptq.py:264 updates everything at once).   */
int crb_set_trailing_lookahead(int mode);

/* The same look-ahead inside crb_hinv_upper_factor: after a 1024-column outer panel only the next
 * panel's columns of the trailing matrix are updated on the caller's stream, the rest on a side
 * stream beside the next panel's chain of diagonal blocks.  Bit-identical factor.  Default on
 * (C > 2048); returns the previous setting.                                                    */
int crb_set_factor_lookahead(int enable);

/* ---- self-test of the bounded waits -----------------------------------------------
 * Every wait inside the tensor-core kernels gives up after a time limit, raises
 * CRB_FLAG_WAIT_LIMIT in the status word, drains its copies, frees its tensor memory and
 * returns (the counterpart of the reference's only failure handling, the retry / fallback
 * around torch.linalg.cholesky, bigptq.py:115-126, for a failure that cannot occur in eager
 * PyTorch: a stalled producer).  This call exercises that path without faulting anything:
 * it launches one GEMM tile whose producer warp withholds its loads and whose waits are
 * limited to `limit_us` microseconds; afterwards *status_dev has CRB_FLAG_WAIT_LIMIT set and
 * the context is intact.  scratch_dev: at least 256 KiB of device memory, 256-byte aligned. */
int crb_selftest_wait_limit(void *scratch_dev, size_t scratch_bytes, unsigned limit_us,
                            unsigned *status_dev, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CRB_B200_H */
