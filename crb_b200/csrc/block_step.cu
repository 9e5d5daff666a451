// Block step of the CRB / BiLLM calibration loop for one 128-column block.
//
// Reference path restated here (paths inside the reference project):
//   bigptq.py:142-263          block loop body (masks, three group quantisations, Q/Err/Losses)
//   utils/structure.py:8-20    Hessian metric  M = w^2 / diag(U)^2
//   utils/autosearch.py:28-83  salient-count search (49 candidates) and split search (81)
//   utils/mask.py:7-18         low / mid masks from the split value
//   binary.py:18-39            braq residual binarizer (also the evaluator of both searches)
//   binary.py:577-687          crbog,  binary.py:1544-1638  crb (v7)
//
// Kernel sequence per block (stream ordered, no host synchronisation, no kernel waits on
// another CTA: grid-wide decisions are taken by whichever CTA finishes last):
//   k_metric_colscore  M, column scores, top-50 columns
//   k_sort_rows        every metric row sorted (bitonic network) with its column ids
//   k_salient_search_sorted  49 candidates x rows from prefix sums of the sorted rows, first strict minimum
//   k_select_l1        histogram of the upper 15 key bits of |M|: the bins that hold the 162 order
//                      statistics numpy.quantile(method="linear") interpolates between
//   k_select_collect   the elements of those bins, gathered bin by bin
//   k_select_bins      exact selection inside each bin (two 8-bit levels), the 81 interpolated values
//   k_split_search_sorted  81 candidates x rows from prefix sums of the sorted rows
//   k_finalize         masks, the technique's binarizer per group, Q, Err, Losses
#include <math.h>

#include "common.cuh"

namespace crb {

// float32 bit patterns of torch.linspace(0.10, 0.90, 81) (utils/autosearch.py:65).
__constant__ unsigned c_split_probs[kSplits] = {
    0x3dcccccdu, 0x3de147aeu, 0x3df5c290u, 0x3e051eb8u, 0x3e0f5c29u, 0x3e19999au,
    0x3e23d70au, 0x3e2e147bu, 0x3e3851ecu, 0x3e428f5cu, 0x3e4ccccdu, 0x3e570a3du,
    0x3e6147aeu, 0x3e6b851fu, 0x3e75c28fu, 0x3e800000u, 0x3e851eb8u, 0x3e8a3d71u,
    0x3e8f5c29u, 0x3e947ae1u, 0x3e99999au, 0x3e9eb852u, 0x3ea3d70au, 0x3ea8f5c2u,
    0x3eae147bu, 0x3eb33333u, 0x3eb851ebu, 0x3ebd70a4u, 0x3ec28f5cu, 0x3ec7ae14u,
    0x3ecccccdu, 0x3ed1eb85u, 0x3ed70a3du, 0x3edc28f6u, 0x3ee147aeu, 0x3ee66666u,
    0x3eeb851eu, 0x3ef0a3d7u, 0x3ef5c28fu, 0x3efae147u, 0x3f000000u, 0x3f028f5cu,
    0x3f051eb8u, 0x3f07ae14u, 0x3f0a3d70u, 0x3f0ccccdu, 0x3f0f5c29u, 0x3f11eb85u,
    0x3f147ae1u, 0x3f170a3du, 0x3f199999u, 0x3f1c28f5u, 0x3f1eb852u, 0x3f2147aeu,
    0x3f23d70au, 0x3f266666u, 0x3f28f5c2u, 0x3f2b851eu, 0x3f2e147bu, 0x3f30a3d7u,
    0x3f333333u, 0x3f35c28fu, 0x3f3851ebu, 0x3f3ae147u, 0x3f3d70a4u, 0x3f400000u,
    0x3f428f5cu, 0x3f451eb8u, 0x3f47ae14u, 0x3f4a3d70u, 0x3f4cccccu, 0x3f4f5c29u,
    0x3f51eb85u, 0x3f547ae1u, 0x3f570a3du, 0x3f599999u, 0x3f5c28f5u, 0x3f5eb852u,
    0x3f6147aeu, 0x3f63d70au, 0x3f666666u};

constexpr int kL1Bins = 32768;   // key bits 30..16
constexpr int kL1Smem = (kL1Bins + kL1Bins / 32) * (int)sizeof(unsigned);   // padded, see k_select_l1
__host__ __device__ constexpr int pad1(int b) { return b + (b >> 5); }
constexpr int kMaxCtas1 = 148;   // CTAs of the metric kernel (one per SM at most)
constexpr int kMaxTiles = 512;   // row tiles of the search kernels
constexpr int kAccSlots = 136;   // 0..48 salient candidates, 49..129 split candidates, 130 salient-group term
constexpr int kAccSplit = kSalCand, kAccSalTerm = kSalCand + kSplits;
static_assert(kAccSalTerm < kAccSlots, "accumulator slots");

// Device workspace of the block step, carved by carve_block_ws().
struct BlockWs {
    unsigned* status;        // [16]   persistent status word (+ padding)
    // ---- zeroed before every block (one memset) ----
    unsigned char* zero_begin;
    size_t zero_bytes;
    unsigned* counters;      // [16]   last-CTA tickets, one per kernel
    unsigned* hist1;         // [kL1Bins]
    unsigned char* slot1;    // [kL1Bins] 0 = not a target bin, else level-1 slot + 1
    unsigned* cursor;        // [kTargets] fill level of each target bin's list
    unsigned* barrier;       // [16]   arrival counters of the grid barriers of k_select_fused
    unsigned long long* acc; // [kAccSlots] fixed-point candidate error sums (49 salient, 81 split, 1 salient term)
    // ---- scratch ----
    float* M;                // [R][128] metric
    float* sv;               // [R][128] every row of M sorted ascending
    unsigned char* sc;       // [R][128] the column of each sorted value
    double* colpart;         // [kMaxCtas1][128]
    double* energy;          // [kMaxCtas1] per-CTA sum of M^2 (bounds every candidate error)
    double* fx;              // [2] fixed-point scale of the error sums and its inverse
    unsigned char* rank;     // [128] position of each column in the score order (>= 50: never salient)
    int* sel;                // [8]   0: i*   1: k*   2: number of target bins (lists)
    float* pvals;            // [kSplits + 1]  the 81 split candidates, [81] = chosen split
    unsigned* tgt_rank;      // [kTargets]
    unsigned* tgt_bin1;      // [kTargets]
    unsigned* tgt_rem;       // [kTargets] rank left inside the target's level-1 bin
    unsigned* tgt_slot;      // [kTargets] index of the target's bin among the target bins (its list)
    float* tgt_frac;         // [kSplits]  interpolation weight
    unsigned* list_off;      // [kTargets + 1] per level-1 slot: start of its list (elements, zeros excluded)
    unsigned* tgt_val;       // [kTargets] bit pattern of each order statistic
    unsigned short* list;    // [R * 128] low 16 key bits of the elements that fall into a target bin, slot by slot
    double* trace_dummy;     // [CRB_TRACE_DOUBLES] sink when the caller passes no trace
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static size_t carve_block_ws(void* base, int R, BlockWs* ws) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void* p = base ? static_cast<char*>(base) + off : nullptr;
        off += align_up(bytes, 256);
        return p;
    };
    BlockWs w;
    w.status = static_cast<unsigned*>(take(64));
    const size_t z0 = off;
    w.counters = static_cast<unsigned*>(take(64));
    w.hist1 = static_cast<unsigned*>(take(sizeof(unsigned) * kL1Bins));
    w.slot1 = static_cast<unsigned char*>(take(kL1Bins));
    w.cursor = static_cast<unsigned*>(take(sizeof(unsigned) * kTargets));
    w.barrier = static_cast<unsigned*>(take(64));
    w.acc = static_cast<unsigned long long*>(take(sizeof(unsigned long long) * kAccSlots));
    w.zero_begin = base ? static_cast<unsigned char*>(base) + z0 : nullptr;
    w.zero_bytes = off - z0;
    w.M = static_cast<float*>(take(sizeof(float) * (size_t)R * kBlock));
    w.sv = static_cast<float*>(take(sizeof(float) * (size_t)R * kBlock));
    w.sc = static_cast<unsigned char*>(take((size_t)R * kBlock));
    w.colpart = static_cast<double*>(take(sizeof(double) * kMaxCtas1 * kBlock));
    w.energy = static_cast<double*>(take(sizeof(double) * kMaxCtas1));
    w.fx = static_cast<double*>(take(sizeof(double) * 2));
    w.rank = static_cast<unsigned char*>(take(kBlock));
    w.sel = static_cast<int*>(take(sizeof(int) * 8));
    w.pvals = static_cast<float*>(take(sizeof(float) * (kSplits + 1)));
    w.tgt_rank = static_cast<unsigned*>(take(sizeof(unsigned) * kTargets));
    w.tgt_bin1 = static_cast<unsigned*>(take(sizeof(unsigned) * kTargets));
    w.tgt_rem = static_cast<unsigned*>(take(sizeof(unsigned) * kTargets));
    w.tgt_slot = static_cast<unsigned*>(take(sizeof(unsigned) * kTargets));
    w.tgt_frac = static_cast<float*>(take(sizeof(float) * kSplits));
    w.list_off = static_cast<unsigned*>(take(sizeof(unsigned) * (kTargets + 1)));
    w.tgt_val = static_cast<unsigned*>(take(sizeof(unsigned) * kTargets));
    w.list = static_cast<unsigned short*>(take(sizeof(unsigned short) * (size_t)R * kBlock));
    w.trace_dummy = static_cast<double*>(take(sizeof(double) * CRB_TRACE_DOUBLES));
    if (ws) *ws = w;
    return off;
}

// ---------------------------------------------------------------------------------------
// Row sort: every row of the metric sorted ascending together with the column of each value
// (bitonic network, one warp per row, four elements per lane; ties keep the lower column first).
// The sorted rows turn the candidate evaluations of both searches into prefix-sum lookups.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ bool key_less(unsigned ka, int ca, unsigned kb, int cb) {
    return (ka < kb) || (ka == kb && ca < cb);
}

__device__ __forceinline__ void sort_metric_row(const float* __restrict__ M, int row, float* __restrict__ sv,
                                                unsigned char* __restrict__ sc, int lane) {
    unsigned k[4];
    int c[4];
    {
        const float4 v = *reinterpret_cast<const float4*>(M + (int64_t)row * kBlock + 4 * lane);
        // keys that order like the values, negative ones included (the magnitude metric is the
        // signed weight): flip all bits of a negative number, the sign bit of the others
        k[0] = ordered_key(v.x); k[1] = ordered_key(v.y); k[2] = ordered_key(v.z); k[3] = ordered_key(v.w);
#pragma unroll
        for (int q = 0; q < 4; ++q) c[q] = 4 * lane + q;
    }
#pragma unroll
    for (int size = 2; size <= kBlock; size <<= 1) {
#pragma unroll
        for (int j = size >> 1; j >= 1; j >>= 1) {
            if (j >= 4) {
                const int lj = j >> 2;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int e = 4 * lane + q;
                    const unsigned ok = __shfl_xor_sync(0xffffffffu, k[q], lj);
                    const int oc = __shfl_xor_sync(0xffffffffu, c[q], lj);
                    const bool up = (e & size) == 0;            // ascending segment
                    const bool lower_half = (e & j) == 0;       // this element keeps the smaller key
                    const bool mine_less = key_less(k[q], c[q], ok, oc);
                    const bool keep = (lower_half == up) ? mine_less : !mine_less;
                    if (!keep) { k[q] = ok; c[q] = oc; }
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int qq = q ^ j;
                    if (qq > q) {
                        const int e = 4 * lane + q;
                        const bool up = (e & size) == 0;
                        const bool in_order = key_less(k[q], c[q], k[qq], c[qq]);
                        if (in_order != up) {
                            const unsigned tk = k[q]; k[q] = k[qq]; k[qq] = tk;
                            const int tc = c[q]; c[q] = c[qq]; c[qq] = tc;
                        }
                    }
                }
            }
        }
    }
    *reinterpret_cast<float4*>(sv + (int64_t)row * kBlock + 4 * lane) =
        make_float4(key_value(k[0]), key_value(k[1]), key_value(k[2]), key_value(k[3]));
    *reinterpret_cast<uchar4*>(sc + (int64_t)row * kBlock + 4 * lane) =
        make_uchar4((unsigned char)c[0], (unsigned char)c[1], (unsigned char)c[2], (unsigned char)c[3]);
}

// One warp per row, eight rows per CTA: many small CTAs, because a single row's network is a
// chain of dependent shuffles (fused into the metric kernel, whose grid is at most one CTA per SM,
// the sort took 10 us longer per block at 4096 rows and 70 us longer at 16384).
__global__ void __launch_bounds__(256)
k_sort_rows(const float* __restrict__ M, int R, float* __restrict__ sv, unsigned char* __restrict__ sc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    chain_wait();
    if (row < R) sort_metric_row(M, row, sv, sc, lane);
}

// ---------------------------------------------------------------------------------------
// K1: metric, column scores, top-50 columns                     (structure.py:10, autosearch.py:37-42)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_metric_colscore(const float* __restrict__ W, int R, int64_t ldw, int col0,
                  const float* __restrict__ U, int64_t ldu, int rows_per_cta, int metric,
                  float* __restrict__ M, double* __restrict__ colpart, double* __restrict__ energy,
                  double* __restrict__ fx, unsigned* counters, unsigned char* __restrict__ rank_out,
                  double* __restrict__ trace, unsigned* status, uint4* __restrict__ zero_ptr, int zero_vecs) {
    __shared__ float s_d2[kBlock];
    __shared__ double s_e[8];
    __shared__ double s_wcol[8][kBlock];
    __shared__ double s_score[kBlock];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = row_in_warp(lane), l = lane_in_row(lane);
    chain_wait();
    // histograms and accumulators of the later kernels of this block step start at zero: cleared
    // here instead of by a separate memset node in front of every block
    for (int k = blockIdx.x * blockDim.x + tid; k < zero_vecs; k += gridDim.x * blockDim.x)
        zero_ptr[k] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kBlock) {
        const float d = U[(int64_t)(col0 + tid) * ldu + col0 + tid];
        s_d2[tid] = __fmul_rn(d, d);
    }
    __syncthreads();
    float d2[16], csum[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) { d2[j] = s_d2[col_of(l, j)]; csum[j] = 0.f; }
    bool bad = false;
    double e2 = 0.0;
    const int row_base = blockIdx.x * rows_per_cta;
    for (int p = 0; p < rows_per_cta; p += 32) {
        const int row = row_base + p + warp * 4 + g;
        if (row < R && row < row_base + rows_per_cta) {
            float x[16];
            load_row16(W + (int64_t)row * ldw + col0, l, x);
            float e = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                // structure.py:10-12: w^2 / diag(U)^2 (hessian) or the weight itself (magnitude)
                const float m = (metric == CRB_METRIC_HESSIAN) ? __fdiv_rn(__fmul_rn(x[j], x[j]), d2[j]) : x[j];
                bad |= !isfinite(m);
                x[j] = m;
                csum[j] += fabsf(m);   // column score = sum of |M| (autosearch.py:37)
                e = fmaf(m, m, e);
            }
            e2 += (double)e;
            store_row16(M + (int64_t)row * kBlock, l, x);
        }
    }
    e2 = warp_sum_d(e2);
    if (lane == 0) s_e[warp] = e2;
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, CRB_FLAG_NONFINITE);

    // sum the 4 rows of the warp, then the 8 warps, in double
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        double v = (double)csum[j];
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (g == 0) s_wcol[warp][col_of(l, j)] = v;
    }
    __syncthreads();
    if (tid < kBlock) {
        double v = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += s_wcol[w][tid];
        colpart[(size_t)blockIdx.x * kBlock + tid] = v;
    }
    if (tid == 0) {
        double v = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += s_e[w];
        energy[blockIdx.x] = v;
    }
    if (!last_cta_done(&counters[0], gridDim.x)) return;

    {
        // column scores: two threads per column, each over half of the CTAs' partial sums, many
        // independent loads in flight (this tail runs on one SM and is bound by load latency)
        const int col = tid & (kBlock - 1), half = tid >> 7;
        const unsigned per = (gridDim.x + 1) / 2;
        const unsigned c0 = half * per, c1 = min(gridDim.x, c0 + per);
        double v = 0.0;
#pragma unroll 16
        for (unsigned c = c0; c < c1; ++c) v += __ldcg(&colpart[(size_t)c * kBlock + col]);
        s_wcol[half][col] = v;
    }
    __syncthreads();
    if (tid < kBlock) s_score[tid] = s_wcol[0][tid] + s_wcol[1][tid];
    if (warp == 4) {
        // Candidate error sums are accumulated as 64-bit fixed point so that their value does not
        // depend on the order in which CTAs add to them.  No candidate error exceeds sum(M^2):
        // scale it to 2^61.
        double v = 0.0;
        for (unsigned c = lane; c < gridDim.x; c += 32) v += __ldcg(&energy[c]);
        v = warp_sum_d(v);
        if (lane == 0) {
            int ex = 0;
            if (v > 0.0 && isfinite(v)) frexp(v, &ex);
            fx[0] = ldexp(1.0, 61 - ex);
            fx[1] = ldexp(1.0, ex - 61);
        }
    }
    __syncthreads();
    if (tid < kBlock) {
        const double mine = s_score[tid];
        int r = 0;
        for (int c = 0; c < kBlock; ++c) {
            const double o = s_score[c];
            r += (o > mine) || (o == mine && c < tid);
        }
        rank_out[tid] = (unsigned char)r;
        if (r < kSalLimit) { trace[6 + r] = (double)tid; trace[267 + r] = mine; }
    }
}

// ---------------------------------------------------------------------------------------
// Helpers shared by the two searches
// ---------------------------------------------------------------------------------------
// Adds a non-negative float64 partial sum to a fixed-point accumulator (order independent).
__device__ __forceinline__ void acc_add(unsigned long long* acc, double v, double scale) {
    const unsigned long long q = __double2ull_rn(fmax(v, 0.0) * scale);
    if (q) atomicAdd(acc, q);
}

// First strict minimum (autosearch.py:53, :78) and the relative gap to the runner-up, taken by
// one full warp (candidates strided over the lanes); NaN never wins, `fallback` if nothing does.
__device__ void warp_first_strict_min(const double* e, int n, int fallback, int* best_out, double* gap_out) {
    const int lane = threadIdx.x & 31;
    double be = INFINITY;
    int best = 0x7fffffff;
    for (int c = lane; c < n; c += 32)
        if (e[c] < be) { be = e[c]; best = c; }            // lowest index of the lane's minimum
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double ov = __shfl_xor_sync(0xffffffffu, be, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best, o);
        if (ov < be || (ov == be && oi < best)) { be = ov; best = oi; }
    }
    const bool none = !(be < INFINITY);
    double second = INFINITY;
    for (int c = lane; c < n; c += 32)
        if (c != best && e[c] < second) second = e[c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) second = fmin(second, __shfl_xor_sync(0xffffffffu, second, o));
    *best_out = none ? fallback : best;
    *gap_out = (none || !(be > 0.0)) ? 0.0 : (second - be) / be;
}

// ---------------------------------------------------------------------------------------
// K3-K5: exact selection of the order statistics behind the 81 quantiles
// (autosearch.py:62-68: numpy.quantile of |M * ~mask3| flattened, zeros at salient columns
// included).  Keys are the float bit patterns of |M|.  A histogram of the upper 15 key bits finds
// the bins that hold the targets; the elements of those bins (typically a fifth of the block) are
// gathered bin by bin as 16-bit remainders and each bin is searched on its own with two 8-bit
// histograms.  The salient zeros are added to bin 0 as a count.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned block_exclusive_scan_1024(unsigned v, unsigned* s_warp) {
    // exclusive scan of one value per thread over a 1024-thread CTA
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned w = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        s_warp[lane] = w;   // inclusive scan of the warp totals
    }
    __syncthreads();
    const unsigned base = warp ? s_warp[warp - 1] : 0u;
    return base + inc - v;
}

// The selection runs either as three kernels (k_select_l1 / k_select_collect / k_select_bins, each
// handing over through the last CTA that finishes) or as one cooperative kernel whose CTAs meet at
// grid barriers (k_select_fused); both are built from the phases below.

// Phase 1: histogram of key bits 30..16 over the non-salient elements this CTA reads, merged into
// the global histogram.  Bin b lives at s_hist[pad1(b)]: one spare word per 32 bins, so that the
// scan of phase 2, in which every thread walks its own 32 consecutive bins, is free of bank conflicts.
__device__ __forceinline__ void select_histogram(const float* __restrict__ M, int R, const bool* s_sal,
                                                 unsigned* s_hist, const BlockWs& ws, int cta, int nctas) {
    const int tid = threadIdx.x;
    const size_t n4 = (size_t)R * (kBlock / 4);
    for (size_t idx = (size_t)cta * blockDim.x + tid; idx < n4; idx += (size_t)nctas * blockDim.x) {
        const int c4 = (int)(idx & 31) * 4;
        const float4 v = *reinterpret_cast<const float4*>(M + idx * 4);
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (!s_sal[c4 + k]) atomicAdd(&s_hist[pad1(__float_as_uint(vv[k]) >> 16 & (kL1Bins - 1))], 1u);
    }
    __syncthreads();
    for (int k = tid; k < kL1Bins; k += blockDim.x) {
        const unsigned c = s_hist[pad1(k)];
        if (c) atomicAdd(&ws.hist1[k], c);
    }
}

// Phase 2 (one CTA of 1024 threads): prefix of the global histogram, the bin of each of the 162 target
// ranks, the target bins numbered in rank order and the start of each one's list.
__device__ void select_locate(int R, int isal, unsigned* s_hist, const BlockWs& ws) {
    __shared__ unsigned s_warp[32];
    __shared__ unsigned s_tbin[kTargets];
    __shared__ unsigned s_trank[kTargets];
    const int tid = threadIdx.x;
    // ---- scan + locate the 162 target ranks ----
    const unsigned N = (unsigned)R * kBlock;
    const unsigned zeros = (unsigned)R * (unsigned)isal;
    {
        // 32768 counters as 8 independent 16-byte loads per thread
        const uint4* src = reinterpret_cast<const uint4*>(ws.hist1);
        uint4 h[kL1Bins / 4 / 1024];
#pragma unroll
        for (int u = 0; u < kL1Bins / 4 / 1024; ++u) h[u] = __ldcg(&src[tid + 1024 * u]);
#pragma unroll
        for (int u = 0; u < kL1Bins / 4 / 1024; ++u) {
            const int b = pad1(4 * (tid + 1024 * u));                // four bins of one 32-bin group
            s_hist[b] = h[u].x; s_hist[b + 1] = h[u].y; s_hist[b + 2] = h[u].z; s_hist[b + 3] = h[u].w;
        }
        __syncthreads();
        if (tid == 0) s_hist[0] += zeros;
    }
    __syncthreads();
    {
        // exclusive prefix over all bins: thread t owns bins 32 t .. 32 t + 31 (words 33 t ..)
        unsigned loc = 0;
        unsigned* mine = s_hist + tid * 33;
#pragma unroll 8
        for (int k = 0; k < 32; ++k) loc += mine[k];
        unsigned run = block_exclusive_scan_1024(loc, s_warp);
#pragma unroll 8
        for (int k = 0; k < 32; ++k) { const unsigned c = mine[k]; mine[k] = run; run += c; }
    }
    __syncthreads();
    if (tid < kSplits) {
        // numpy: virtual index (N-1)*p in float32, floor, fractional weight in float32
        const float p = __uint_as_float(c_split_probs[tid]);
        const float vi = __fmul_rn((float)(N - 1), p);
        const float lo = floorf(vi);
        ws.tgt_frac[tid] = __fsub_rn(vi, lo);
        const unsigned ilo = (unsigned)lo;
        s_trank[2 * tid] = min(ilo, N - 1);
        s_trank[2 * tid + 1] = min(ilo + 1, N - 1);
    }
    __syncthreads();
    if (tid < kTargets) {
        const unsigned r = s_trank[tid];
        ws.tgt_rank[tid] = r;
        int lo = 0, hi = kL1Bins;                 // last bin with exclusive prefix <= r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_hist[pad1(mid)] <= r) lo = mid; else hi = mid;
        }
        s_tbin[tid] = (unsigned)lo;
        ws.tgt_bin1[tid] = (unsigned)lo;
        ws.tgt_rem[tid] = r - s_hist[pad1(lo)];
    }
    __syncthreads();
    // level-1 slots: the number of distinct bins before each target (targets are rank ordered); per
    // slot the start of its list in the collection buffer (the bin's element count is exact: it is
    // the difference of two prefix values, less the salient zeros that are only counted)
    if (tid < 32) {
        unsigned base = 0;
        for (int t0 = 0; t0 < kTargets; t0 += 32) {
            const int t = t0 + tid;
            const bool fresh = t < kTargets && t > 0 && s_tbin[t] != s_tbin[t - 1];
            const unsigned m = __ballot_sync(0xffffffffu, fresh);
            if (t < kTargets) {
                const unsigned slot = base + __popc(m & (0xffffffffu >> (31 - tid)));
                ws.tgt_slot[t] = slot;
                if (fresh || t == 0) {
                    const unsigned bin = s_tbin[t];
                    ws.slot1[bin] = (unsigned char)(slot + 1);
                    const unsigned next = (bin + 1 < (unsigned)kL1Bins) ? s_hist[pad1(bin + 1)] : N;
                    s_trank[slot] = next - s_hist[pad1(bin)] - (bin == 0 ? zeros : 0u);   // reused: count per slot
                }
                if (t == kTargets - 1) ws.sel[2] = (int)slot + 1;
            }
            base += __popc(m);
        }
        __syncwarp();
        // exclusive scan of the (at most 162) slot counts
        const unsigned nslot = base + 1;
        unsigned run = 0;
        for (unsigned s0 = 0; s0 < nslot; s0 += 32) {
            const unsigned sidx = s0 + tid;
            const unsigned c = sidx < nslot ? s_trank[sidx] : 0u;
            unsigned inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned v = __shfl_up_sync(0xffffffffu, inc, o);
                if (tid >= o) inc += v;
            }
            if (sidx < nslot) ws.list_off[sidx] = run + inc - c;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (tid == 0) ws.list_off[nslot] = run;
    }
}

// Phase 3: the low 16 key bits of every non-salient element that falls into a target bin, appended
// to that bin's list (exact-size segments, order irrelevant).  A CTA first counts its elements per
// list in shared memory, reserves one range per list with a single global atomic, then writes.
__device__ __forceinline__ void select_collect(const float* __restrict__ M, int R, const bool* s_sal,
                                               const BlockWs& ws, int cta, int nctas) {
    __shared__ unsigned s_cnt[kTargets], s_base[kTargets];
    const int tid = threadIdx.x;
    if (tid < kTargets) s_cnt[tid] = 0u;
    __syncthreads();
    const size_t n4 = (size_t)R * (kBlock / 4);
    const size_t first = (size_t)cta * blockDim.x + tid, stride = (size_t)nctas * blockDim.x;
    for (size_t idx = first; idx < n4; idx += stride) {
        const int c4 = (int)(idx & 31) * 4;
        const float4 v = *reinterpret_cast<const float4*>(M + idx * 4);
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (s_sal[c4 + k]) continue;
            const unsigned s1 = ws.slot1[(__float_as_uint(vv[k]) & 0x7fffffffu) >> 16];
            if (s1) atomicAdd(&s_cnt[s1 - 1], 1u);
        }
    }
    __syncthreads();
    if (tid < kTargets) {
        const unsigned c = s_cnt[tid];
        s_base[tid] = c ? ws.list_off[tid] + atomicAdd(&ws.cursor[tid], c) : 0u;
        s_cnt[tid] = 0u;
    }
    __syncthreads();
    for (size_t idx = first; idx < n4; idx += stride) {
        const int c4 = (int)(idx & 31) * 4;
        const float4 v = *reinterpret_cast<const float4*>(M + idx * 4);
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (s_sal[c4 + k]) continue;
            const unsigned key = __float_as_uint(vv[k]) & 0x7fffffffu;
            const unsigned s1 = ws.slot1[key >> 16];
            if (!s1) continue;
            const unsigned pos = atomicAdd(&s_cnt[s1 - 1], 1u);
            ws.list[s_base[s1 - 1] + pos] = (unsigned short)(key & 0xffffu);
        }
    }
}

// Phase 4: selection inside one target bin.  The bin's list holds the low 16 key bits of its
// elements; every target of the bin (usually one to four) is located by two 8-bit histogram levels
// over that list.  The histogram of the high byte is shared by all targets of the bin, the one of
// the low byte by all targets with the same high byte.  Any CTA size from 256 to 1024 threads.
__device__ void select_in_bin(int R, int isal, int slot, const BlockWs& ws) {
    __shared__ unsigned s_hi[256], s_lo[256], s_scan[256], s_warp[32];
    __shared__ int s_t0, s_t1;
    __shared__ unsigned s_pick, s_left;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned nthreads = blockDim.x;
    const bool owner = tid < 256;                            // one thread per histogram counter
    // exclusive scan over the CTA of one counter per thread (zero beyond the first 256 threads)
    auto scan_cta = [&](unsigned v) {
        unsigned inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) s_warp[warp] = inc;
        __syncthreads();
        unsigned base = 0;
        for (int w = 0; w < warp; ++w) base += s_warp[w];
        __syncthreads();
        return base + inc - v;
    };
    if (tid == 0) { s_t0 = kTargets; s_t1 = -1; }
    __syncthreads();
    if (tid < kTargets && (int)ws.tgt_slot[tid] == slot) { atomicMin(&s_t0, tid); atomicMax(&s_t1, tid); }
    const unsigned off = ws.list_off[slot], n = ws.list_off[slot + 1] - off;
    const unsigned short* list = ws.list + off;
    if (owner) s_hi[tid] = 0u;
    __syncthreads();
    const int t0 = s_t0, t1 = s_t1;
    const unsigned bin1 = ws.tgt_bin1[t0];
    const unsigned zeros = bin1 == 0u ? (unsigned)R * (unsigned)isal : 0u;   // salient zeros: counted, not listed
    for (unsigned k = tid; k < n; k += nthreads) atomicAdd(&s_hi[__ldcg(list + k) >> 8], 1u);
    __syncthreads();
    const unsigned hi_cnt = owner ? s_hi[tid] : 0u;
    const unsigned hi_exc = scan_cta(hi_cnt);
    int lo_of = -1;                                      // high byte the low-byte histogram currently describes
    for (int t = t0; t <= t1; ++t) {
        unsigned rem = ws.tgt_rem[t];
        if (rem < zeros) {                               // one of the counted zeros: the value is 0
            if (tid == 0) ws.tgt_val[t] = 0u;
            continue;
        }
        rem -= zeros;
        if (hi_exc <= rem && rem < hi_exc + hi_cnt) { s_pick = (unsigned)tid; s_left = rem - hi_exc; }
        __syncthreads();
        const unsigned hi = s_pick, left = s_left;
        if ((int)hi != lo_of) {
            if (owner) s_lo[tid] = 0u;
            __syncthreads();
            for (unsigned k = tid; k < n; k += nthreads) {
                const unsigned e = __ldcg(list + k);
                if ((e >> 8) == hi) atomicAdd(&s_lo[e & 255u], 1u);
            }
            __syncthreads();
            const unsigned exc = scan_cta(owner ? s_lo[tid] : 0u);
            if (owner) s_scan[tid] = exc;
            lo_of = (int)hi;
            __syncthreads();
        }
        if (owner) {
            const unsigned lo_cnt = s_lo[tid], lo_exc = s_scan[tid];
            if (lo_exc <= left && left < lo_exc + lo_cnt) ws.tgt_val[t] = (bin1 << 16) | (hi << 8) | (unsigned)tid;
        }
        __syncthreads();
    }
    __syncthreads();
}

// The 81 split candidates from the 162 order statistics, exactly as numpy interpolates them.
__device__ __forceinline__ void select_interpolate(const BlockWs& ws) {
    const int tid = threadIdx.x;
    if (tid < kSplits) {
        // numpy _lerp: a + (b-a)*t, replaced by b - (b-a)*(1-t) when t >= 0.5; float32, unfused
        const float a = __uint_as_float(__ldcg(&ws.tgt_val[2 * tid])), b = __uint_as_float(__ldcg(&ws.tgt_val[2 * tid + 1]));
        const float t = ws.tgt_frac[tid];
        const float diff = __fsub_rn(b, a);
        const float v0 = __fadd_rn(a, __fmul_rn(diff, t));
        const float v1 = __fsub_rn(b, __fmul_rn(diff, __fsub_rn(1.0f, t)));
        ws.pvals[tid] = (t >= 0.5f) ? v1 : v0;
    }
}

__global__ void __launch_bounds__(1024)
k_select_l1(const float* __restrict__ M, int R, const unsigned char* __restrict__ rank,
            const int* __restrict__ sel, BlockWs ws) {
    extern __shared__ __align__(16) unsigned s_hist[];   // kL1Smem bytes
    __shared__ bool s_sal[kBlock];
    const int tid = threadIdx.x;
    for (int k = tid; k < kL1Bins + kL1Bins / 32; k += blockDim.x) s_hist[k] = 0u;
    chain_wait();
    const int isal = sel[0];
    if (tid < kBlock) s_sal[tid] = rank[tid] < isal;
    __syncthreads();
    select_histogram(M, R, s_sal, s_hist, ws, blockIdx.x, gridDim.x);
    if (!last_cta_done(&ws.counters[2], gridDim.x)) return;
    select_locate(R, isal, s_hist, ws);
}

__global__ void __launch_bounds__(1024)
k_select_collect(const float* __restrict__ M, int R, const unsigned char* __restrict__ rank,
                 const int* __restrict__ sel, BlockWs ws) {
    __shared__ bool s_sal[kBlock];
    const int tid = threadIdx.x;
    chain_wait();
    const int isal = sel[0];
    if (tid < kBlock) s_sal[tid] = rank[tid] < isal;
    __syncthreads();
    select_collect(M, R, s_sal, ws, blockIdx.x, gridDim.x);
}

constexpr int kBinThreads = 512;
__global__ void __launch_bounds__(kBinThreads)
k_select_bins(int R, const int* __restrict__ sel, BlockWs ws) {
    chain_wait();
    if ((int)blockIdx.x < sel[2]) select_in_bin(R, sel[0], blockIdx.x, ws);
    if (!last_cta_done(&ws.counters[3], gridDim.x)) return;
    select_interpolate(ws);
}

// All CTAs of a cooperative launch meet here.  The wait is bounded: a CTA that gives up raises
// CRB_FLAG_WAIT_LIMIT and the kernel returns (every CTA then runs out the same way).
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned expected, unsigned* status) {
    __shared__ int s_ok;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd(counter, 1u);
        int ok = 0;
        for (unsigned it = 0; it < (1u << 22); ++it) {       // each probe is a round trip to L2: seconds in all
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= expected) { ok = 1; break; }
        }
        if (!ok) atomicOr(status, CRB_FLAG_WAIT_LIMIT);
        s_ok = ok;
    }
    __syncthreads();
    return s_ok != 0;
}

// The three selection kernels as one cooperative launch (one CTA per SM at most, all resident).
__global__ void __launch_bounds__(1024)
k_select_fused(const float* __restrict__ M, int R, const unsigned char* __restrict__ rank,
               const int* __restrict__ sel, BlockWs ws) {
    extern __shared__ __align__(16) unsigned s_hist[];   // kL1Smem bytes
    __shared__ bool s_sal[kBlock];
    const int tid = threadIdx.x;
    const unsigned nctas = gridDim.x;
    for (int k = tid; k < kL1Bins + kL1Bins / 32; k += blockDim.x) s_hist[k] = 0u;
    const int isal = sel[0];
    if (tid < kBlock) s_sal[tid] = rank[tid] < isal;
    __syncthreads();
    select_histogram(M, R, s_sal, s_hist, ws, blockIdx.x, nctas);
    if (!grid_barrier(&ws.barrier[0], nctas, ws.status)) return;
    if (blockIdx.x == 0) select_locate(R, isal, s_hist, ws);
    if (!grid_barrier(&ws.barrier[1], nctas, ws.status)) return;
    select_collect(M, R, s_sal, ws, blockIdx.x, nctas);
    if (!grid_barrier(&ws.barrier[2], nctas, ws.status)) return;
    const int nslot = __ldcg(&ws.sel[2]);
    for (int slot = blockIdx.x; slot < nslot; slot += nctas) select_in_bin(R, isal, slot, ws);
    if (!last_cta_done(&ws.counters[3], nctas)) return;
    select_interpolate(ws);
}

// ---------------------------------------------------------------------------------------
// K6: split search on sorted rows                                      (autosearch.py:72-81)
//
// Per row the non-salient values are kept sorted with float64 prefix sums of x and x^2.  A split
// candidate p cuts the row at c = #{x < p}; each side is a contiguous range [a, b) whose order-1
// expansion (binary.py:18-39) follows from prefix sums:  mu = sum / m;  the elements below mu are
// [a, cm), so  A = sum|x - mu| = mu (cm - a) - S[a,cm) + S[cm,b) - mu (b - cm),  alpha = A / m,
// squared error = sum (x - mu)^2 - 2 alpha A + m alpha^2.  mu and alpha are rounded to float32
// where the reference holds them in float32; everything else is float64, which is at least as
// accurate as the reference's float32 element-wise evaluation (differences ~1e-7 relative).
// One thread per (row, candidate); three binary searches per task.
// ---------------------------------------------------------------------------------------
constexpr int kSplitRows = 8;                    // rows per pass of a CTA (small: more CTAs in flight, the phases are latency bound)
constexpr int kRowPitch = kBlock + 1;            // odd pitch: rows start in different banks
constexpr int kSplitSmem = kSplitRows * kRowPitch * (int)(sizeof(float) + 2 * sizeof(double)) +
                           (kSplits + 1) * kSplitRows * (int)sizeof(double);

__device__ __forceinline__ int lower_bound_f(const float* v, int a, int b, float t) {
    int lo = a, len = b - a;                     // first index in [a, b) with v[idx] >= t
    while (len > 0) {
        const int half = len >> 1;
        if (v[lo + half] < t) { lo += half + 1; len -= half + 1; } else { len = half; }
    }
    return lo;
}

// squared error of the one-expansion binarizer on the sorted range [a, b) of one row
__device__ __forceinline__ double range_order1_err(const float* v, const double* P1, const double* P2, int a, int b) {
    const int m = b - a;
    if (m <= 0) return 0.0;
    const double S1 = P1[b] - P1[a], S2 = P2[b] - P2[a];
    const float mu_f = __fdiv_rn((float)S1, (float)m);
    const double mu = (double)mu_f;
    const int cm = lower_bound_f(v, a, b, mu_f);
    const double below = P1[cm] - P1[a];
    const double A = mu * (double)(cm - a) - below + (S1 - below) - mu * (double)(b - cm);
    const double alpha = (double)__fdiv_rn((float)A, (float)m);
    return S2 - 2.0 * mu * S1 + (double)m * mu * mu - 2.0 * alpha * A + (double)m * alpha * alpha;
}

// The same for the union of two sorted ranges [a0, b0) and [a1, b1), a0 <= b0 <= a1 <= b1: with the
// magnitude metric the values are signed and the "mid" side |x| >= p is the two tails of the row.
__device__ __forceinline__ double two_range_order1_err(const float* v, const double* P1, const double* P2, int n,
                                                       int a0, int b0, int a1, int b1) {
    const int m = (b0 - a0) + (b1 - a1);
    if (m <= 0) return 0.0;
    const double S1 = (P1[b0] - P1[a0]) + (P1[b1] - P1[a1]);
    const double S2 = (P2[b0] - P2[a0]) + (P2[b1] - P2[a1]);
    const float mu_f = __fdiv_rn((float)S1, (float)m);
    const double mu = (double)mu_f;
    const int cm = lower_bound_f(v, 0, n, mu_f);                  // members below mu: the part of each range in front of cm
    const int c0 = min(max(cm, a0), b0), c1 = min(max(cm, a1), b1);
    const double below = (P1[c0] - P1[a0]) + (P1[c1] - P1[a1]);
    const double nb = (double)((c0 - a0) + (c1 - a1));
    const double A = mu * nb - below + (S1 - below) - mu * ((double)m - nb);
    const double alpha = (double)__fdiv_rn((float)A, (float)m);
    return S2 - 2.0 * mu * S1 + (double)m * mu * mu - 2.0 * alpha * A + (double)m * alpha * alpha;
}

// first index in [0, n) with v[idx] > t
__device__ __forceinline__ int upper_bound_f(const float* v, int n, float t) {
    int lo = 0, len = n;
    while (len > 0) {
        const int half = len >> 1;
        if (!(v[lo + half] > t)) { lo += half + 1; len -= half + 1; } else { len = half; }
    }
    return lo;
}

__global__ void __launch_bounds__(256)
k_split_search_sorted(const float* __restrict__ sv, const unsigned char* __restrict__ sc, int R,
                      int rows_per_cta, int metric, const unsigned char* __restrict__ rank,
                      const float* __restrict__ pvals_in, unsigned long long* __restrict__ acc,
                      const double* __restrict__ fx, unsigned* counters, int* __restrict__ sel,
                      float* __restrict__ pvals_out, double* __restrict__ trace, unsigned* status) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    double* s_P1 = reinterpret_cast<double*>(s_raw);                         // [rows][pitch]
    double* s_P2 = s_P1 + kSplitRows * kRowPitch;
    double* s_acc = s_P2 + kSplitRows * kRowPitch;                           // [kSplits + 1][rows]
    float* s_v = reinterpret_cast<float*>(s_acc + (kSplits + 1) * kSplitRows);   // [rows][pitch]
    __shared__ float s_p[kSplits];
    __shared__ unsigned char s_rank[kBlock];
    __shared__ double s_tot[kSplits + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int k = tid; k < (kSplits + 1) * kSplitRows; k += blockDim.x) s_acc[k] = 0.0;
    chain_wait();
    const int isal = sel[0];
    const int n = kBlock - isal;                                             // non-salient values per row
    if (tid < kSplits) s_p[tid] = pvals_in[tid];
    if (tid < kBlock) s_rank[tid] = rank[tid];
    __syncthreads();

    const int row_base = blockIdx.x * rows_per_cta;
    for (int p0 = 0; p0 < rows_per_cta; p0 += kSplitRows) {
        // ---- phase A: one warp per row: drop the salient columns, keep the order, prefix sums ----
        for (int r = warp; r < kSplitRows; r += 8) {
            const int row = row_base + p0 + r;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            bool ns[4] = {false, false, false, false};
            if (row < R) {
                const float4 v = *reinterpret_cast<const float4*>(sv + (int64_t)row * kBlock + 4 * lane);
                const uchar4 c = *reinterpret_cast<const uchar4*>(sc + (int64_t)row * kBlock + 4 * lane);
                x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
                ns[0] = s_rank[c.x] >= isal; ns[1] = s_rank[c.y] >= isal;
                ns[2] = s_rank[c.z] >= isal; ns[3] = s_rank[c.w] >= isal;
            }
            // salient-group term (order-2 expansion on the isal salient values of the row), by the warp
            {
                const float ds = (float)max(isal, 1);
                float s = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) s += (row < R && !ns[q]) ? x[q] : 0.f;
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                const float mu = __fdiv_rn(s, ds);
                float dv[4], a = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) { dv[q] = x[q] - mu; a += (row < R && !ns[q]) ? fabsf(dv[q]) : 0.f; }
                for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                const float al = __fdiv_rn(a, ds);
                float y1[4];
                s = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    y1[q] = __fadd_rn(al * sgnf(dv[q]), mu);
                    dv[q] = x[q] - y1[q];
                    s += (row < R && !ns[q]) ? dv[q] : 0.f;
                }
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                const float mu2 = __fdiv_rn(s, ds);
                a = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) { dv[q] -= mu2; a += (row < R && !ns[q]) ? fabsf(dv[q]) : 0.f; }
                for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                const float al2 = __fdiv_rn(a, ds);
                float e = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float qv = __fadd_rn(y1[q], __fadd_rn(al2 * sgnf(dv[q]), mu2));
                    const float d = x[q] - qv;
                    e += (row < R && !ns[q]) ? d * d : 0.f;
                }
                for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
                if (lane == 0) s_acc[kSplits * kSplitRows + r] += (double)e;
            }
            // compaction: position of each kept value = number of kept values before it
            const int mine = (int)ns[0] + (int)ns[1] + (int)ns[2] + (int)ns[3];
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            int pos = incl - mine;
            float* vrow = s_v + r * kRowPitch;
            double l1 = 0.0, l2 = 0.0;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (ns[q]) { vrow[pos++] = x[q]; l1 += (double)x[q]; l2 += (double)x[q] * (double)x[q]; }
            // exclusive float64 scan of the per-lane sums, then the running prefix inside the lane
            double i1 = l1, i2 = l2;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t1 = __shfl_up_sync(0xffffffffu, i1, o);
                const double t2 = __shfl_up_sync(0xffffffffu, i2, o);
                if (lane >= o) { i1 += t1; i2 += t2; }
            }
            double r1 = i1 - l1, r2 = i2 - l2;
            double* P1 = s_P1 + r * kRowPitch;
            double* P2 = s_P2 + r * kRowPitch;
            pos = incl - mine;
            if (lane == 0) { P1[0] = 0.0; P2[0] = 0.0; }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (ns[q]) {
                    r1 += (double)x[q]; r2 += (double)x[q] * (double)x[q];
                    ++pos;
                    P1[pos] = r1; P2[pos] = r2;
                }
        }
        __syncthreads();
        // ---- phase B: one thread per (row, candidate) ----
        for (int task = tid; task < kSplitRows * kSplits; task += blockDim.x) {
            const int r = task % kSplitRows, k = task / kSplitRows;
            if (row_base + p0 + r >= R) continue;
            const float* v = s_v + r * kRowPitch;
            const double* P1 = s_P1 + r * kRowPitch;
            const double* P2 = s_P2 + r * kRowPitch;
            double e;
            if (metric == CRB_METRIC_HESSIAN) {
                const int c = lower_bound_f(v, 0, n, s_p[k]);               // low side: x < p (mask.py:11-13), x >= 0
                e = range_order1_err(v, P1, P2, 0, c) + range_order1_err(v, P1, P2, c, n);
            } else {
                // signed values: low side |x| < p is the middle of the sorted row, mid side its two tails
                const int b = lower_bound_f(v, 0, n, s_p[k]);
                const int a = min(upper_bound_f(v, n, -s_p[k]), b);         // p = 0: nothing is below it
                e = range_order1_err(v, P1, P2, a, b) + two_range_order1_err(v, P1, P2, n, 0, a, b, n);
            }
            s_acc[k * kSplitRows + r] += e;
        }
        __syncthreads();
    }
    if (tid <= kSplits) {
        double t = 0.0;
#pragma unroll 8
        for (int r = 0; r < kSplitRows; ++r) t += s_acc[tid * kSplitRows + r];
        acc_add(&acc[kAccSplit + tid], t, fx[0]);        // slot kAccSplit + 81 is the salient-group term
    }
    if (!last_cta_done(&counters[5], gridDim.x)) return;

    if (tid <= kSplits) s_tot[tid] = (double)__ldcg(&acc[kAccSplit + tid]) * fx[1];
    __syncthreads();
    const double e3 = s_tot[kSplits];
    __syncthreads();
    if (tid < kSplits) s_tot[tid] += e3;
    __syncthreads();
    const double inv = 1.0 / ((double)R * kBlock);
    if (tid < kSplits) {
        trace[105 + tid] = s_tot[tid] * inv;
        trace[186 + tid] = (double)s_p[tid];
        if (!isfinite(s_tot[tid])) atomicOr(status, CRB_FLAG_NONFINITE);
    }
    if (warp == 0) {
        int best; double gap;
        warp_first_strict_min(s_tot, kSplits, kSplits / 2, &best, &gap);
        if (lane == 0) {
            sel[1] = best;
            const float p = s_p[best];
            pvals_out[kSplits] = p;
            trace[1] = (double)best;
            trace[2] = (double)p;
            trace[4] = gap;
            trace[5] = e3 * inv;
        }
    }
}

// ---------------------------------------------------------------------------------------
// K2: salient-count search on sorted rows                              (autosearch.py:44-55)
//
// Candidate i moves the i highest-score columns into the salient set S_i.  Per row:
//  * S_i (at most 49 values, kept in score order) is evaluated directly;
//  * the complement is the whole sorted row minus those i values ("holes"): any count / sum /
//    sum of squares below a threshold is a prefix-sum lookup on the whole row minus a pass over
//    the holes.  The order-2 expansion (binary.py:18-39) needs three thresholds: mu1, and the
//    second-pass split points y1 + mu2 of the elements below / above mu1.
// One thread per (row, candidate); the 32 lanes of a warp share the candidate, so the hole
// loops have the same length across the warp.
// ---------------------------------------------------------------------------------------
constexpr int kSalRows = 16;
constexpr int kTopPitch = kSalLimit + 1;
constexpr int kSalSmem = kSalRows * kRowPitch * (int)(sizeof(float) + 2 * sizeof(double)) +
                         kSalRows * kTopPitch * (int)(2 * sizeof(float) + 3 * sizeof(double)) +
                         kSalCand * kSalRows * (int)sizeof(double);

// Smallest float that is not below t.  For a float x:  x < t  <=>  x < float_not_below(t), and
// x >= t  <=>  x >= float_not_below(t): comparisons of float data with a double threshold can
// be made in float without changing a single outcome (and without a conversion per element).
__device__ __forceinline__ float float_not_below(double t) { return __double2float_ru(t); }

// The hole passes and the direct float32 evaluation of the i top values walk the same list: they
// are fused pairwise (four passes over tv[0..i) in all; the plain sums come from per-row running
// sums in score order).
__device__ __forceinline__ double salient_candidate_err(const float* v, const double* P1, const double* P2,
                                                        const float* tv, const double* tvd, const double* hp1,
                                                        const double* hp2, const float* fs, int i) {
    const int n = kBlock - i;
    const float fi = (float)i;
    // sums of the i holes (complement) and of the salient values: running sums in score order,
    // prepared once per row
    const double H1 = hp1[i], H2 = hp2[i];
    float s = fs[i];
    const double S1 = P1[kBlock] - H1, S2 = P2[kBlock] - H2;
    const float mu1 = __fdiv_rn((float)S1, (float)n);
    const float mu = __fdiv_rn(s, fi);
    int cf = lower_bound_f(v, 0, kBlock, mu1);
    int n1 = cf;                                            // elements below mu1 (whole row, then minus holes)
    double a1 = P1[cf], b1 = P2[cf];
    // pass 1: holes below mu1; first scale of the salient group
    float a = 0.f;
#pragma unroll 4
    for (int h = 0; h < i; ++h) {
        const float t = tv[h];
        if (t < mu1) { const double td = tvd[h]; --n1; a1 -= td; b1 = fma(-td, td, b1); }
        a += fabsf(t - mu);
    }
    const double c1 = (double)n1;
    const float al = __fdiv_rn(a, fi);
    const double dmu1 = (double)mu1, dn = (double)n;
    const double A1 = dmu1 * c1 - a1 + (S1 - a1) - dmu1 * (dn - c1);
    const float al1 = __fdiv_rn((float)A1, (float)n);
    const float ylo = __fadd_rn(-al1, mu1), yhi = __fadd_rn(al1, mu1);
    const double sr = (a1 - c1 * (double)ylo) + ((S1 - a1) - (dn - c1) * (double)yhi);
    const float mu2 = __fdiv_rn((float)sr, (float)n);
    const double tlo = (double)ylo + (double)mu2, thi = (double)yhi + (double)mu2;
    const double t1 = fmin(tlo, dmu1), t2 = fmax(thi, dmu1);
    const float f1 = float_not_below(t1), f2 = float_not_below(t2);
    cf = lower_bound_f(v, 0, kBlock, f1);
    int n2 = cf;
    double a2 = P1[cf];
    cf = lower_bound_f(v, 0, kBlock, f2);
    int n3 = cf;
    double a3 = P1[cf];
    // pass 2: holes below the second-pass thresholds; residual mean of the salient group
    s = 0.f;
#pragma unroll 4
    for (int h = 0; h < i; ++h) {
        const float x = tv[h];
        if (x < f1) { --n2; a2 -= tvd[h]; }
        if (x < f2) { --n3; a3 -= tvd[h]; }
        s += x - __fadd_rn(al * sgnf(x - mu), mu);
    }
    const double c2 = (double)n2;
    const double c3 = (double)(n3 - n1);                    // elements in [mu1, t2)
    a3 -= a1;
    const double cu = dn - c1, au = S1 - a1, bu = S2 - b1;  // the group at or above mu1
    const double A2 = (tlo * c2 - a2 + (a1 - a2) - tlo * (c1 - c2)) + (thi * c3 - a3 + (au - a3) - thi * (cu - c3));
    const double al2 = (double)__fdiv_rn((float)A2, (float)n);
    const double SS = (b1 - 2.0 * tlo * a1 + c1 * tlo * tlo) + (bu - 2.0 * thi * au + cu * thi * thi);
    const double err = SS - 2.0 * al2 * A2 + dn * al2 * al2;
    // passes 3 and 4: the i top columns themselves, evaluated like the reference in float32
    const float m2 = __fdiv_rn(s, fi);
    a = 0.f;
#pragma unroll 4
    for (int h = 0; h < i; ++h) a += fabsf((tv[h] - __fadd_rn(al * sgnf(tv[h] - mu), mu)) - m2);
    const float al2s = __fdiv_rn(a, fi);
    float e = 0.f;
#pragma unroll 4
    for (int h = 0; h < i; ++h) {
        const float y1 = __fadd_rn(al * sgnf(tv[h] - mu), mu);
        const float r = (tv[h] - y1) - m2;
        const float d = tv[h] - __fadd_rn(y1, __fadd_rn(al2s * sgnf(r), m2));
        e = fmaf(d, d, e);
    }
    return err + (double)e;
}

// Which candidates (salient counts) a thread evaluates: thread t works on row t % 16 of the tile
// with schedule slot t / 16.  A candidate costs about i + 8 units; the slots are balanced
// (longest-processing-time order).  With 32 slots (512 threads, at most two candidates per
// thread: 51..57 units) a CTA has twice the warps to hide the latency of the dependent
// shared-memory searches than with 16 slots (256 threads, 94..108 units per thread).
#ifndef CRB_SAL_SLOTS
#define CRB_SAL_SLOTS 32
#endif
constexpr int kSalSlots = CRB_SAL_SLOTS;
constexpr int kSalThreads = kSalRows * kSalSlots;
#if CRB_SAL_SLOTS == 16
__constant__ unsigned char c_sal_sched[16][4] = {
    {49, 18, 17, 0}, {48, 19, 16, 0}, {47, 20, 15, 0}, {46, 21, 14, 0}, {45, 22, 13, 0}, {44, 23, 12, 0},
    {43, 24, 11, 0}, {42, 25, 10, 0}, {41, 26, 9, 0}, {40, 27, 8, 0}, {39, 28, 7, 0}, {38, 29, 6, 0},
    {37, 30, 5, 0}, {36, 31, 4, 0}, {35, 32, 3, 0}, {34, 33, 2, 1}};
#else
__constant__ unsigned char c_sal_sched[32][4] = {
    {49, 0, 0, 0}, {48, 0, 0, 0}, {47, 0, 0, 0}, {46, 0, 0, 0}, {45, 0, 0, 0}, {44, 0, 0, 0}, {43, 0, 0, 0},
    {42, 0, 0, 0}, {41, 0, 0, 0}, {40, 0, 0, 0}, {39, 0, 0, 0}, {38, 0, 0, 0}, {37, 0, 0, 0}, {36, 0, 0, 0},
    {35, 0, 0, 0}, {34, 1, 0, 0}, {33, 2, 0, 0}, {32, 3, 0, 0}, {31, 4, 0, 0}, {30, 5, 0, 0}, {29, 6, 0, 0},
    {28, 7, 0, 0}, {27, 8, 0, 0}, {26, 9, 0, 0}, {25, 10, 0, 0}, {24, 11, 0, 0}, {23, 12, 0, 0}, {22, 13, 0, 0},
    {21, 14, 0, 0}, {20, 15, 0, 0}, {19, 16, 0, 0}, {18, 17, 0, 0}};
#endif
static_assert(kSalRows == 16 && kSalCand == 49 && (kSalSlots == 16 || kSalSlots == 32),
              "c_sal_sched is laid out for 16 rows x 16 or 32 slots and 49 candidates");

__global__ void __launch_bounds__(kSalThreads)
k_salient_search_sorted(const float* __restrict__ sv, const unsigned char* __restrict__ sc, int R,
                        int rows_per_cta, const unsigned char* __restrict__ rank,
                        unsigned long long* __restrict__ acc, const double* __restrict__ fx,
                        unsigned* counters, int* __restrict__ sel, double* __restrict__ trace,
                        unsigned* status) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    double* s_P1 = reinterpret_cast<double*>(s_raw);                         // [rows][pitch]
    double* s_P2 = s_P1 + kSalRows * kRowPitch;
    double* s_acc = s_P2 + kSalRows * kRowPitch;                             // [kSalCand][rows]
    float* s_v = reinterpret_cast<float*>(s_acc + kSalCand * kSalRows);      // [rows][pitch]
    float* s_tv = s_v + kSalRows * kRowPitch;                                // [rows][kTopPitch]
    float* s_fs = s_tv + kSalRows * kTopPitch;                               // [rows][kTopPitch] float32 running sum
    double* s_hp1 = reinterpret_cast<double*>(s_fs + kSalRows * kTopPitch);  // [rows][kTopPitch] running sum
    double* s_hp2 = s_hp1 + kSalRows * kTopPitch;                            // [rows][kTopPitch] running sum of squares
    double* s_tvd = s_hp2 + kSalRows * kTopPitch;                            // [rows][kTopPitch] the top values as doubles
    __shared__ unsigned char s_rank[kBlock];
    __shared__ double s_tot[kSalCand];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int k = tid; k < kSalCand * kSalRows; k += blockDim.x) s_acc[k] = 0.0;
    chain_wait();
    if (tid < kBlock) s_rank[tid] = rank[tid];
    __syncthreads();
    const int row_base = blockIdx.x * rows_per_cta;
    for (int p0 = 0; p0 < rows_per_cta; p0 += kSalRows) {
        // ---- phase A: one warp per row: sorted values, float64 prefix sums, top-column values ----
        for (int r = warp; r < kSalRows; r += kSalThreads / 32) {
            const int row = row_base + p0 + r;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            uchar4 c = make_uchar4(0, 0, 0, 0);
            if (row < R) {
                const float4 v = *reinterpret_cast<const float4*>(sv + (int64_t)row * kBlock + 4 * lane);
                c = *reinterpret_cast<const uchar4*>(sc + (int64_t)row * kBlock + 4 * lane);
                x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
            }
            const unsigned char cc[4] = {c.x, c.y, c.z, c.w};
            float* vrow = s_v + r * kRowPitch;
            double l1 = 0.0, l2 = 0.0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                vrow[4 * lane + q] = x[q];
                l1 += (double)x[q]; l2 += (double)x[q] * (double)x[q];
                const int rk = s_rank[cc[q]];
                if (row < R && rk < kSalLimit) {
                    s_tv[r * kTopPitch + rk] = x[q];
                    s_tvd[r * kTopPitch + rk] = (double)x[q];
                }
            }
            double i1 = l1, i2 = l2;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t1 = __shfl_up_sync(0xffffffffu, i1, o);
                const double t2 = __shfl_up_sync(0xffffffffu, i2, o);
                if (lane >= o) { i1 += t1; i2 += t2; }
            }
            double r1 = i1 - l1, r2 = i2 - l2;
            double* P1 = s_P1 + r * kRowPitch;
            double* P2 = s_P2 + r * kRowPitch;
            if (lane == 0) { P1[0] = 0.0; P2[0] = 0.0; }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                r1 += (double)x[q]; r2 += (double)x[q] * (double)x[q];
                P1[4 * lane + q + 1] = r1; P2[4 * lane + q + 1] = r2;
            }
            // running sums of the top-column values in score order ([i] = the first i of them):
            // three lanes, one sequential sum each (the float32 one in the order a plain loop adds)
            __syncwarp();
            if (lane < 3) {
                const float* tvr = s_tv + r * kTopPitch;
                if (lane == 0) {
                    float f = 0.f;
                    float* o = s_fs + r * kTopPitch;
                    o[0] = 0.f;
                    for (int h = 0; h < kSalCand; ++h) { f += tvr[h]; o[h + 1] = f; }
                } else {
                    double d = 0.0;
                    double* o = (lane == 1 ? s_hp1 : s_hp2) + r * kTopPitch;
                    o[0] = 0.0;
                    for (int h = 0; h < kSalCand; ++h) {
                        const double t = (double)tvr[h];
                        d += (lane == 1) ? t : t * t;
                        o[h + 1] = d;
                    }
                }
            }
        }
        __syncthreads();
        // ---- phase B: one thread per (row, schedule slot) ----
        {
            const int r = tid & (kSalRows - 1), slot = tid >> 4;
            if (row_base + p0 + r < R) {
#pragma unroll 1
                for (int k = 0; k < 4; ++k) {
                    const int i = c_sal_sched[slot][k];
                    if (i == 0) break;
                    s_acc[(i - 1) * kSalRows + r] += salient_candidate_err(
                        s_v + r * kRowPitch, s_P1 + r * kRowPitch, s_P2 + r * kRowPitch, s_tv + r * kTopPitch,
                        s_tvd + r * kTopPitch, s_hp1 + r * kTopPitch, s_hp2 + r * kTopPitch, s_fs + r * kTopPitch, i);
                }
            }
        }
        __syncthreads();
    }
    if (tid < kSalCand) {
        double t = 0.0;
#pragma unroll 8
        for (int r = 0; r < kSalRows; ++r) t += s_acc[tid * kSalRows + r];
        acc_add(&acc[tid], t, fx[0]);
    }
    if (!last_cta_done(&counters[1], gridDim.x)) return;

    if (tid < kSalCand) s_tot[tid] = (double)__ldcg(&acc[tid]) * fx[1];
    __syncthreads();
    if (tid < kSalCand) {
        trace[56 + tid] = s_tot[tid] * (1.0 / ((double)R * kBlock));
        if (!isfinite(s_tot[tid])) atomicOr(status, CRB_FLAG_NONFINITE);
    }
    if (warp == 0) {
        int best; double gap;
        warp_first_strict_min(s_tot, kSalCand, max(1, kSalLimit / 3) - 1, &best, &gap);
        if (lane == 0) {
            sel[0] = best + 1;
            trace[0] = (double)(best + 1);
            trace[3] = gap;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Group binarizers on one row held by 8 lanes (16 values per lane, `in` = membership).
// Shared by the block step (K7) and by the stand-alone Binarization.quantize entry point.
// (binary.py:18-39 braq, 577-687 crbog, 1544-1638 crb)
// ---------------------------------------------------------------------------------------
// CRB v7 joint scale solve (binary.py:1582-1596), float32 like the reference.
// `symdamp` damps the correlation whatever its sign (the crb_symdamp variants, binary.py:1584-1587).
__device__ __forceinline__ void crb_solve(float c12, float c1w, float c2w, float d, float lam,
                                          float corr_damp, bool symdamp, float* a1, float* a2) {
    if (symdamp || c12 > 0.f) c12 = __fmul_rn(c12, __fsub_rn(1.0f, corr_damp));
    const float A = __fadd_rn(d, lam);
    const float den = __fsub_rn(__fmul_rn(A, A), __fmul_rn(c12, c12));
    const bool ok = fabsf(den) > 1e-12f;
    const float dn = ok ? den : 1.0f;
    const float x1 = fmaxf(__fdiv_rn(__fsub_rn(__fmul_rn(A, c1w), __fmul_rn(c12, c2w)), dn), 0.f);
    const float x2 = fmaxf(__fdiv_rn(__fsub_rn(__fmul_rn(A, c2w), __fmul_rn(c12, c1w)), dn), 0.f);
    *a1 = ok ? x1 : 0.f;
    *a2 = ok ? x2 : 0.f;
}

// One expansion: q = mu + alpha * sign(w - mu) on the members.  The three techniques share
// this arithmetic (binary.py:24-36, 595-630, 1570-1576).  n = member count of the row.
__device__ __forceinline__ void group_order1(const float (&w)[16], const bool (&in)[16], int n,
                                             float (&q)[16], int (&b1)[16], float* mu_out,
                                             float* al_out) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) s += in[j] ? w[j] : 0.f;
    s = red8(s);
    const float nf = (float)n;
    const float mu = n ? __fdiv_rn(s, nf) : 0.f;
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) a += in[j] ? fabsf(w[j] - mu) : 0.f;
    a = red8(a);
    const float al = n ? __fdiv_rn(a, nf) : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j)
        if (in[j]) {
            const float sg = sgnf(w[j] - mu);
            q[j] = __fadd_rn(al * sg, mu);
            b1[j] = (int)sg;
        }
    *mu_out = mu;
    *al_out = al;
}

// Two expansions with the technique's coupling.  sc[0..3] receives the row's scales:
// braq mu1, alpha1, mu2, alpha2;  crbog mu, alpha1, alpha2, 0;  crb mu + mu_fix, alpha1, alpha2, 0.
__device__ __forceinline__ void group_order2(const float (&w)[16], const bool (&in)[16], int n,
                                             int technique, float lam, float corr_damp,
                                             float (&q)[16], int (&b1)[16], int (&b2)[16],
                                             float (&sc)[4]) {
    const float d = (float)n;
    const float ds = fmaxf(d, 1.0f);                  // rows without members produce nothing
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) s += in[j] ? w[j] : 0.f;
    const float mu = __fdiv_rn(red8(s), ds);
    float c[16], B1[16], B2[16];
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) { c[j] = in[j] ? (w[j] - mu) : 0.f; a += fabsf(c[j]); B1[j] = sgnf(c[j]); }
    const float a_init = __fdiv_rn(red8(a), ds);
    sc[0] = sc[1] = sc[2] = sc[3] = 0.f;

    if (technique == CRB_TECH_BRAQ) {
        // binary.py:18-39 with order 2
        float y1[16], r[16];
        s = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            y1[j] = __fadd_rn(a_init * B1[j], mu);
            r[j] = in[j] ? (w[j] - y1[j]) : 0.f;
            s += r[j];
        }
        const float mu2 = __fdiv_rn(red8(s), ds);
        a = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { r[j] = in[j] ? (r[j] - mu2) : 0.f; a += fabsf(r[j]); }
        const float al2 = __fdiv_rn(red8(a), ds);
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (in[j]) {
                B2[j] = sgnf(r[j]);
                q[j] = __fadd_rn(y1[j], __fadd_rn(al2 * B2[j], mu2));
                b1[j] = (int)B1[j]; b2[j] = (int)B2[j];
            }
        sc[0] = mu; sc[1] = a_init; sc[2] = mu2; sc[3] = al2;
    } else if (technique == CRB_TECH_CRBOG) {
        // binary.py:644-685: no re-centring of the residual, float64 2x2 solve
        float r[16];
        a = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { r[j] = c[j] - a_init * B1[j]; B2[j] = sgnf(r[j]); a += fabsf(r[j]); }
        float al1 = a_init, al2 = __fdiv_rn(red8(a), ds);
        float f12 = 0.f, f1w = 0.f, f2w = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { f12 += B1[j] * B2[j]; f1w += c[j] * B1[j]; f2w += c[j] * B2[j]; }
        const double c12 = (double)red8(f12), c1w = (double)red8(f1w), c2w = (double)red8(f2w);
        const double D = (double)d;
        const double det = D * D - c12 * c12;
        if (fabs(det) > 1e-12) {
            al1 = (float)fmax((c1w * D - c2w * c12) / det, 0.0);
            al2 = (float)fmax((c2w * D - c1w * c12) / det, 0.0);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (in[j]) {
                q[j] = __fadd_rn(__fadd_rn(mu, __fmul_rn(al1, B1[j])), __fmul_rn(al2, B2[j]));
                b1[j] = (int)B1[j]; b2[j] = (int)B2[j];
            }
        sc[0] = mu; sc[1] = al1; sc[2] = al2;
    } else {
        // CRB v7, binary.py:1598-1636 (d_safe = max(count, 1), A = count + lam); the *_norefine
        // variants stop after the first joint solve (binary.py:1617), the *_symdamp ones damp the
        // correlation symmetrically (dispatch binary.py:2883-2890)
        const bool norefine = technique == CRB_TECH_CRB_NOREFINE || technique == CRB_TECH_CRB_SYMDAMP_NOREFINE;
        const bool symdamp = technique == CRB_TECH_CRB_SYMDAMP || technique == CRB_TECH_CRB_SYMDAMP_NOREFINE;
        float t[16];
        auto centred_sign = [&](float (&B)[16]) {
            float ts = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) ts += t[j];
            const float tm = __fdiv_rn(red8(ts), ds);
#pragma unroll
            for (int j = 0; j < 16; ++j) B[j] = in[j] ? sgnf(t[j] - tm) : 0.f;
        };
        auto dot_c = [&](const float (&B)[16]) {
            float v = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) v += c[j] * B[j];
            return red8(v);
        };
        auto dot_b = [&]() {
            float v = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) v += B1[j] * B2[j];
            return red8(v);
        };
#pragma unroll
        for (int j = 0; j < 16; ++j) t[j] = in[j] ? (c[j] - a_init * B1[j]) : 0.f;
        centred_sign(B2);                                         // step 3
        float c1w = dot_c(B1), c2w = dot_c(B2), a1, a2;
        crb_solve(dot_b(), c1w, c2w, d, lam, corr_damp, symdamp, &a1, &a2);   // step 4
        if (!norefine) {
#pragma unroll
            for (int j = 0; j < 16; ++j) t[j] = in[j] ? (c[j] - a1 * B1[j]) : 0.f;
            centred_sign(B2);                                     // step 5
            c2w = dot_c(B2);
            crb_solve(dot_b(), c1w, c2w, d, lam, corr_damp, symdamp, &a1, &a2);
#pragma unroll
            for (int j = 0; j < 16; ++j) t[j] = in[j] ? (c[j] - a2 * B2[j]) : 0.f;
            centred_sign(B1);                                     // step 6
            c1w = dot_c(B1);
            crb_solve(dot_b(), c1w, c2w, d, lam, corr_damp, symdamp, &a1, &a2);
        }
        float rs = 0.f;                                           // step 7
#pragma unroll
        for (int j = 0; j < 16; ++j)
            rs += in[j] ? (c[j] - __fadd_rn(__fmul_rn(a1, B1[j]), __fmul_rn(a2, B2[j]))) : 0.f;
        const float mu_fix = __fdiv_rn(red8(rs), ds);
        const float base = __fadd_rn(mu, mu_fix);
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (in[j]) {
                q[j] = __fadd_rn(__fadd_rn(base, __fmul_rn(a1, B1[j])), __fmul_rn(a2, B2[j]));
                b1[j] = (int)B1[j]; b2[j] = (int)B2[j];
            }
        sc[0] = base; sc[1] = a1; sc[2] = a2;
    }
}

// ---------------------------------------------------------------------------------------
// K7: final masks, the technique's binarizer on the three groups, Q / Err / Losses
// (bigptq.py:246-263)
// ---------------------------------------------------------------------------------------
// kDefaultOrders: the reference's default orders = (1, 1, 2), compiled without the per-group
// order dispatch (the generic form costs about a third more time in this kernel).
// kMinCtas: 1 lets the compiler keep everything in registers (190 per thread, one CTA per SM):
// best while the grid has at most one CTA per SM anyway (up to 4736 rows); 2 caps the registers at
// 128 (a few spills) so that two CTAs share an SM: 3 % faster per block at 16384 rows.
template <bool kDefaultOrders, int kMinCtas>
__global__ void __launch_bounds__(256, kMinCtas)
k_finalize(float* __restrict__ W, int R, int64_t ldw, int col0, const float* __restrict__ U,
           int64_t ldu, const unsigned char* __restrict__ rank, const int* __restrict__ sel,
           const float* __restrict__ pvals, int technique, int orders, int metric, float lam, float corr_damp,
           float* __restrict__ Err, int64_t ld_err, float* __restrict__ Losses,
           unsigned char* __restrict__ codes, int64_t ld_codes, float* __restrict__ scales) {
    __shared__ float s_d[kBlock];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = row_in_warp(lane), l = lane_in_row(lane);
    chain_wait();
    if (tid < kBlock) s_d[tid] = U[(int64_t)(col0 + tid) * ldu + col0 + tid];
    __syncthreads();
    const int isal = sel[0];
    const float psplit = pvals[kSplits];
    const int row = blockIdx.x * 32 + warp * 4 + g;
    const bool live = row < R;
    float w[16], dd[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) dd[j] = s_d[col_of(l, j)];
    if (live) {
        load_row16(W + (int64_t)row * ldw + col0, l, w);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = 0.f;
    }
    // group of every element: 0 low, 1 mid, 2 salient (mask.py:7-18 on the metric); a NaN metric
    // belongs to no group (3) and is reconstructed as 0, as in the reference
    int grp[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float m = (metric == CRB_METRIC_HESSIAN) ? __fdiv_rn(__fmul_rn(w[j], w[j]), __fmul_rn(dd[j], dd[j]))
                                                       : fabsf(w[j]);
        grp[j] = ((int)rank[col_of(l, j)] < isal) ? 2 : ((m < psplit) ? 0 : ((m >= psplit) ? 1 : 3));
    }
    float q[16], sc[8];
    int b1[16], b2[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) { q[j] = 0.f; b1[j] = 0; b2[j] = 0; }
    // expansions per group (bigptq.py:246-247 hands orders[i] to the quantizer): decimal digits of
    // `orders`, 112 = (low 1, mid 1, salient 2), the only combination whose scales fit `sc`
#pragma unroll
    for (int k = 0; k < 8; ++k) sc[k] = 0.f;
    if (kDefaultOrders) {
#pragma unroll
        for (int gi = 0; gi < 2; ++gi) {
            bool in[16];
            int n = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) { in[j] = grp[j] == gi; n += in[j]; }
            n = red8i(n);
            group_order1(w, in, n, q, b1, &sc[2 * gi], &sc[2 * gi + 1]);
        }
        bool in[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) in[j] = grp[j] == 2;
        float s2[4];
        group_order2(w, in, isal, technique, lam, corr_damp, q, b1, b2, s2);
        sc[4] = s2[0]; sc[5] = s2[1]; sc[6] = s2[2]; sc[7] = s2[3];
    } else
#pragma unroll 1
    for (int gi = 0; gi < 3; ++gi) {
        const int order = (gi == 0) ? orders / 100 : ((gi == 1) ? (orders / 10) % 10 : orders % 10);
        bool in[16];
        int n = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) { in[j] = grp[j] == gi; n += in[j]; }
        n = red8i(n);
        if (order == 1) {
            float mu, al;
            group_order1(w, in, n, q, b1, &mu, &al);
            if (gi == 0) { sc[0] = mu; sc[1] = al; } else if (gi == 1) { sc[2] = mu; sc[3] = al; } else { sc[4] = mu; sc[5] = al; }
        } else {
            float s2[4];
            group_order2(w, in, n, technique, lam, corr_damp, q, b1, b2, s2);
            if (gi == 2) { sc[4] = s2[0]; sc[5] = s2[1]; sc[6] = s2[2]; sc[7] = s2[3]; }
        }
    }

    // ---- column epilogue (bigptq.py:249-263) ----
    float e[16];
    float loss = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float diff = w[j] - q[j];
        e[j] = __fdiv_rn(diff, dd[j]);
        loss += __fdiv_rn(__fmul_rn(diff, diff), __fmul_rn(dd[j], dd[j]));
    }
    loss = red8(loss);
    if (!live) return;
    store_row16(W + (int64_t)row * ldw + col0, l, q);
    store_row16(Err + (int64_t)row * ld_err, l, e);
    if (l == 0) Losses[row] += loss * 0.5f;
    if (codes) {
#pragma unroll
        for (int ee = 0; ee < 4; ++ee) {
            uchar4 cc;
            unsigned char* pc = reinterpret_cast<unsigned char*>(&cc);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int j = 4 * ee + v;
                pc[v] = (unsigned char)((b1[j] + 1) | ((b2[j] + 1) << 2) | ((grp[j] & 3) << 4));
            }
            *reinterpret_cast<uchar4*>(codes + (int64_t)row * ld_codes + col0 + 32 * ee + 4 * l) = cc;
        }
    }
    if (scales && l == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) scales[(int64_t)row * 8 + k] = sc[k];
    }
}

// Stand-alone group binarizer on a [R, 128] block with an arbitrary element mask:
// Binarization.quantize (binary.py:2868-2884) for braq / crbog / crb, order 1 or 2.
__global__ void __launch_bounds__(256)
k_binarize_group(const float* __restrict__ W, int R, int64_t ldw, const unsigned char* __restrict__ mask,
                 int64_t ldm, int order, int technique, float lam, float corr_damp,
                 float* __restrict__ Q, int64_t ldq) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = row_in_warp(lane), l = lane_in_row(lane);
    const int row = blockIdx.x * 32 + warp * 4 + g;
    const bool live = row < R;
    float w[16], q[16];
    bool in[16];
    int b1[16], b2[16];
    int n = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) { w[j] = 0.f; q[j] = 0.f; in[j] = false; b1[j] = 0; b2[j] = 0; }
    if (live) {
        load_row16(W + (int64_t)row * ldw, l, w);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uchar4 m = *reinterpret_cast<const uchar4*>(mask + (int64_t)row * ldm + 32 * e + 4 * l);
            in[4 * e + 0] = m.x != 0; in[4 * e + 1] = m.y != 0; in[4 * e + 2] = m.z != 0; in[4 * e + 3] = m.w != 0;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) n += in[j];
    }
    n = red8i(n);
    if (order == 1) {
        float mu, al;
        group_order1(w, in, n, q, b1, &mu, &al);
    } else {
        float sc[4];
        group_order2(w, in, n, technique, lam, corr_damp, q, b1, b2, sc);
    }
    if (live) store_row16(Q + (int64_t)row * ldq, l, q);
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static int ceil_div(int a, int b) { return (a + b - 1) / b; }

size_t block_workspace_bytes(int R) { return carve_block_ws(nullptr, R, nullptr); }

// `orders`: expansions of the low / mid / salient group as decimal digits (112 = the reference's
// default orders=(1, 1, 2), bigptq.py:56); each digit 1 or 2.
bool orders_valid(int orders) {
    const int a = orders / 100, b = orders / 10 % 10, c = orders % 10;
    return orders > 0 && orders < 1000 && (a == 1 || a == 2) && (b == 1 || b == 2) && (c == 1 || c == 2);
}

int block_step_launch(float* W, int R, int64_t ldw, const float* U, int64_t ldu, int block,
                      int technique, int orders, float lam, float corr_damp, int metric, float* Err, int64_t ld_err,
                      float* Losses, unsigned char* codes, int64_t ld_codes, float* scales,
                      double* trace, void* workspace, size_t workspace_bytes, cudaStream_t st, bool reset_tickets) {
    if (!W || !U || !Err || !Losses || !workspace || R <= 0 || block < 0) return CRB_ERR_BAD_ARG;
    if (ld_err < kBlock || (ld_err & 3)) return CRB_ERR_BAD_ARG;
    if (technique < CRB_TECH_BRAQ || technique > CRB_TECH_CRB_SYMDAMP_NOREFINE) return CRB_ERR_BAD_ARG;
    if (!orders_valid(orders)) return CRB_ERR_BAD_ARG;
    if (orders != CRB_ORDERS_DEFAULT && scales) return CRB_ERR_UNSUPPORTED;   // the 8 scale slots hold (1, 1, 2) only
    if (metric != CRB_METRIC_HESSIAN && metric != CRB_METRIC_MAGNITUDE) return CRB_ERR_BAD_ARG;
    if ((ldw & 3) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(Err) & 15))
        return CRB_ERR_BAD_ARG;
    if ((long long)R * kBlock >= (1ll << 31)) return CRB_ERR_UNSUPPORTED;
    BlockWs ws;
    if (carve_block_ws(workspace, R, &ws) > workspace_bytes) return CRB_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return CRB_ERR_BAD_ARG;
    double* tr = trace ? trace : ws.trace_dummy;
    const int col0 = block * kBlock;

    static PerDeviceSetup once;
    int sm_count = 0;
    int rc_setup = once.run([] {
        if (cudaFuncSetAttribute(k_select_l1, cudaFuncAttributeMaxDynamicSharedMemorySize, kL1Smem) != cudaSuccess ||
            cudaFuncSetAttribute(k_select_fused, cudaFuncAttributeMaxDynamicSharedMemorySize, kL1Smem) != cudaSuccess ||
            cudaFuncSetAttribute(k_split_search_sorted, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSplitSmem) != cudaSuccess ||
            cudaFuncSetAttribute(k_salient_search_sorted, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSalSmem) != cudaSuccess)
            return (int)CRB_ERR_LAUNCH;
        return (int)CRB_OK;
    }, &sm_count);
    if (rc_setup != CRB_OK) return rc_setup;
    // the last-CTA tickets reset themselves; a caller that cannot vouch for them (first use of a
    // workspace, stand-alone calls) asks for a reset
    if (reset_tickets && cudaMemsetAsync(ws.counters, 0, 64, st) != cudaSuccess) return CRB_ERR_LAUNCH;

    // K1
    const int rows1 = 32 * ceil_div(R, 32 * kMaxCtas1);
    launch_chained(k_metric_colscore, ceil_div(R, rows1), 256, 0, st, W, R, ldw, col0, U, ldu, rows1, metric, ws.M, ws.colpart,
                   ws.energy, ws.fx, ws.counters, ws.rank, tr, ws.status,
                   reinterpret_cast<uint4*>(ws.zero_begin + 64), (int)((ws.zero_bytes - 64) / 16));
    CRB_LAUNCHED();
    launch_chained(k_sort_rows, ceil_div(R, 8), 256, 0, st, ws.M, R, ws.sv, ws.sc);
    CRB_LAUNCHED();
    // K2: salient-count search on the sorted rows (<= kMaxTiles CTAs)
    const int rows_sal = kSalRows * ceil_div(R, kSalRows * kMaxTiles);
    launch_chained(k_salient_search_sorted, ceil_div(R, rows_sal), kSalThreads, kSalSmem, st,
                   ws.sv, ws.sc, R, rows_sal, ws.rank, ws.acc, ws.fx, ws.counters, ws.sel, tr, ws.status);
    CRB_LAUNCHED();
    // K3-K5
    const int n4 = R * (kBlock / 4);
    const int g2 = min(148, ceil_div(n4, 1024));
    if (g_fused_selection.load(std::memory_order_relaxed)) {
        // one cooperative launch: all CTAs resident (one per SM: 132 KB of shared memory each)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)min(g2, sm_count > 0 ? sm_count : 1));
        cfg.blockDim = dim3(1024);
        cfg.dynamicSmemBytes = kL1Smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, k_select_fused, (const float*)ws.M, R, (const unsigned char*)ws.rank,
                               (const int*)ws.sel, ws) != cudaSuccess)
            return CRB_ERR_LAUNCH;
        CRB_LAUNCHED();
    } else {
        const int g1 = min(148, ceil_div(n4, 1024 * 4));
        launch_chained(k_select_l1, g1, 1024, kL1Smem, st, ws.M, R, ws.rank, ws.sel, ws);
        CRB_LAUNCHED();
        launch_chained(k_select_collect, g2, 1024, 0, st, ws.M, R, ws.rank, ws.sel, ws);
        CRB_LAUNCHED();
        launch_chained(k_select_bins, kTargets, kBinThreads, 0, st, R, ws.sel, ws);
        CRB_LAUNCHED();
    }
    // K6: split search on the sorted rows
    const int rows_sp = kSplitRows * ceil_div(R, kSplitRows * kMaxTiles);
    launch_chained(k_split_search_sorted, ceil_div(R, rows_sp), 256, kSplitSmem, st,
                   ws.sv, ws.sc, R, rows_sp, metric, ws.rank, ws.pvals, ws.acc, ws.fx, ws.counters, ws.sel, ws.pvals, tr, ws.status);
    CRB_LAUNCHED();
    // K7
    const bool one_wave = ceil_div(R, 32) <= 148;
    auto* finalize = orders == CRB_ORDERS_DEFAULT ? (one_wave ? k_finalize<true, 1> : k_finalize<true, 2>)
                                                  : (one_wave ? k_finalize<false, 1> : k_finalize<false, 2>);
    launch_chained(finalize, ceil_div(R, 32), 256, 0, st,
                   W, R, ldw, col0, U, ldu, ws.rank, ws.sel, ws.pvals, technique,
                   orders, metric, lam, corr_damp, Err, ld_err, Losses, codes, ld_codes, scales);
    CRB_LAUNCHED();
    return CRB_OK;
}

int binarize_group_launch(const float* W, int R, int64_t ldw, const unsigned char* mask, int64_t ldm,
                          int order, int technique, float lam, float corr_damp, float* Q, int64_t ldq,
                          cudaStream_t st) {
    if (!W || !mask || !Q || R <= 0) return CRB_ERR_BAD_ARG;
    if (order != 1 && order != 2) return CRB_ERR_UNSUPPORTED;
    if (technique < CRB_TECH_BRAQ || technique > CRB_TECH_CRB_SYMDAMP_NOREFINE) return CRB_ERR_BAD_ARG;
    if ((ldw & 3) || (ldq & 3) || (ldm & 3) || ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Q)) & 15) ||
        (reinterpret_cast<uintptr_t>(mask) & 3))
        return CRB_ERR_BAD_ARG;
    k_binarize_group<<<ceil_div(R, 32), 256, 0, st>>>(W, R, ldw, mask, ldm, order, technique, lam, corr_damp, Q, ldq);
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
