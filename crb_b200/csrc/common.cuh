// Shared helpers for the crb_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/crb_b200.h"

namespace crb {

// Host-side count of kernels launched by this library (crb_launch_count()); several host
// threads may drive different streams at once.
extern std::atomic<unsigned long long> g_launches;

#define CRB_LAUNCHED()                                   \
    do {                                                 \
        ::crb::g_launches.fetch_add(1, std::memory_order_relaxed); \
        if (cudaGetLastError() != cudaSuccess) return CRB_ERR_LAUNCH; \
    } while (0)

// ---- programmatic dependent launch ------------------------------------------------------
// The path is a long chain of short, stream-ordered kernels (one block step is eight of them,
// one factorisation step three): the gap between two dependent launches is a visible share of
// the chain.  Kernels launched through launch_chained() may be placed on free SMs while their
// predecessor in the stream still runs; each of them calls chain_wait() before it reads or
// writes global memory, which returns only when the predecessor has completed and its writes
// are visible, so stream order is kept for the data.  What overlaps is the launch itself and
// the part of a kernel in front of chain_wait() (shared-memory set-up, barrier and tensor-memory
// allocation).  chain_wait() is a no-op for a kernel launched the ordinary way.
extern std::atomic<int> g_fused_selection;    // 1: quantile selection as one cooperative kernel; crb_set_fused_selection()
extern std::atomic<int> g_dependent_launch;   // 1: use it (default); crb_set_dependent_launch()

#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // from here on the next kernel of the stream may be scheduled next to this one; it blocks in
    // its own chain_wait() until this grid has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_dependent_launch.load(std::memory_order_relaxed) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Per-device one-time set-up.  Function attributes (the dynamic shared-memory limit of a kernel)
// and device properties belong to a DEVICE, not to the process: a host that drives several GPUs
// has to set them once on each.  `run(setup)` calls `setup()` (returning a crbStatus) the first
// time it is reached with a given device current, under a mutex, and reports that device's
// multiprocessor count.
constexpr int kMaxDevices = 64;
struct PerDeviceSetup {
    std::mutex lock;
    bool done[kMaxDevices] = {};
    int sms[kMaxDevices] = {};
    template <class F>
    int run(F setup, int* sm_count = nullptr) {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return CRB_ERR_LAUNCH;
        std::lock_guard<std::mutex> guard(lock);
        if (!done[dev]) {
            const int rc = setup();
            if (rc != CRB_OK) return rc;
            int n = 0;
            if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
            sms[dev] = n;
            done[dev] = true;
        }
        if (sm_count) *sm_count = sms[dev];
        return CRB_OK;
    }
};

constexpr int kBlock = CRB_BLOCK;            // 128 columns per block step
constexpr int kSalLimit = CRB_SALIENT_LIMIT; // 50
constexpr int kSalCand = kSalLimit - 1;      // candidates i = 1..49
constexpr int kSplits = CRB_N_SPLITS;        // 81
constexpr int kTargets = 2 * kSplits;        // order statistics needed by the 81 quantiles

// ---- row layout used by every row-parallel kernel -------------------------------------
// A warp covers 4 rows; the 8 lanes of a row hold 16 columns each: register 4e+v of lane l
// is column 32e + 4l + v, so that one float4 load per e is a 128-byte coalesced segment.
__device__ __forceinline__ int row_in_warp(int lane) { return lane >> 3; }
__device__ __forceinline__ int lane_in_row(int lane) { return lane & 7; }
__device__ __forceinline__ int col_of(int l, int j) { return 32 * (j >> 2) + 4 * l + (j & 3); }

__device__ __forceinline__ float red8(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}
__device__ __forceinline__ int red8i(int v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// torch.sign semantics: sign(0) = 0, sign(NaN) = 0.
__device__ __forceinline__ float sgnf(float v) { return (v > 0.f) ? 1.f : ((v < 0.f) ? -1.f : 0.f); }

// Loads the 16 values of this lane from a row of 128 floats (16-byte aligned).
__device__ __forceinline__ void load_row16(const float* __restrict__ row, int l, float (&x)[16]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float4 v = *reinterpret_cast<const float4*>(row + 32 * e + 4 * l);
        x[4 * e + 0] = v.x; x[4 * e + 1] = v.y; x[4 * e + 2] = v.z; x[4 * e + 3] = v.w;
    }
}
__device__ __forceinline__ void store_row16(float* __restrict__ row, int l, const float (&x)[16]) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
        *reinterpret_cast<float4*>(row + 32 * e + 4 * l) =
            make_float4(x[4 * e + 0], x[4 * e + 1], x[4 * e + 2], x[4 * e + 3]);
}

// "Last CTA done" election: returns true in exactly one CTA of the grid, after every other
// CTA's global writes (made before the call) are visible to it.  No CTA waits on another.
// The ticket counter must be 0 at launch; the elected CTA leaves it at 0 again.
__device__ __forceinline__ bool last_cta_done(unsigned* counter, unsigned total) {
    __shared__ bool s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(counter, 1u);
        s_last = (t == total - 1);
        if (s_last) *counter = 0u;          // nobody else touches it any more: ready for the next launch
    }
    __syncthreads();
    if (s_last) __threadfence();
    return s_last;
}

// A second stream per (device, caller stream) with the caller stream's priority, and a pool of events
// to fork to it and join it again (factor.cu keeps the table).  Used where a chain of small kernels
// on the caller's stream can run beside work that only a later step needs.
struct SideContext {
    cudaStream_t side = nullptr;
    cudaStream_t side2 = nullptr;     // a second one for work that must not queue behind the first
    std::vector<cudaEvent_t> events;
};
SideContext* side_context(cudaStream_t main, size_t n_events);

extern std::atomic<int> g_factor_lookahead;     // 0 off, 1 on (default): look-ahead over the factorisation's rank-1024 updates
extern std::atomic<int> g_trailing_lookahead;   // 0 off, 1 by shape (default), 2 always; crb_set_trailing_lookahead()

// Shape flags of gemm_tf32x3 (gemm_tc.cu).
constexpr int GEMM_LOWER_ONLY = 1;   // write only the 128 x 128 blocks of C on or below the diagonal
constexpr int GEMM_B_LOWER = 2;      // the [K, N] operand B is lower triangular (zero for k < n)
constexpr int GEMM_A_LOWER = 4;      // the [M, K] operand A is lower triangular (zero for k > m)
// `selftest` (normally NULL) shortens the barrier waits and can make the producer warp withhold
// its loads, so that a wait runs out on purpose: the kernel must then raise CRB_FLAG_WAIT_LIMIT,
// drain and return (crb_selftest_wait_limit).
struct GemmSelfTest {
    unsigned long long wait_ns;
    int withhold_loads;
};
int gemm_tf32x3(bool b_is_nk, int shape, int M, int N, int K, float alpha, const float* A, int64_t lda,
                const float* B, int64_t ldb, float beta, float* C, int64_t ldc, unsigned* status,
                cudaStream_t st, const GemmSelfTest* selftest = nullptr, int max_ctas = 0);

}  // namespace crb
