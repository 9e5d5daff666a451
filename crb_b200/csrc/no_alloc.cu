// crb_block_step_static: the block step for callers that cannot hand over a workspace.
//
// Some hosts of this library may not allocate device memory at the moment they need a block
// step: an operator hook that runs inside a serving or training framework which has already
// given the whole GPU to its own memory pool (a cudaMalloc there fails or fragments the pool),
// or a latency-critical loop that cannot afford the device-wide synchronisation a cudaMalloc /
// cudaFree pair implies.  For them this file keeps the scratch memory of the block step inside
// the library image: a file-scope __device__ array that every GPU loading the library holds
// from module load until exit.  The entry point below makes no cudaMalloc, cudaFree or any
// other allocating call; inputs and outputs are still the caller's buffers.
//
// Limits and rules
//   * at most CRB_STATIC_MAX_ROWS (16384) rows per call; larger R is refused with
//     CRB_ERR_STATIC_LIMIT before anything is launched;
//   * the array costs kStaticScratchBytes (23 MiB) of device memory on every GPU that loads
//     the library, whether or not this entry point is ever called;
//   * all calls on a device share the one array.  It keeps whatever the previous call left,
//     so each call clears the parts that must start at zero (status word, tickets,
//     histograms) on the caller's stream before its kernels run.  Two calls that overlap on
//     the GPU (different streams, or different host threads without ordering) race on the
//     array and give undefined results: serialise them;
//   * the first call on each device resolves the device address of the array
//     (cudaGetSymbolAddress, with that device current); with lazy module loading this is
//     also the call that places the library's device code and the array on that GPU, so the
//     promise of no allocation holds from the second call on.  Make that first call outside
//     any stream capture.
#include <mutex>

#include "common.cuh"

namespace crb {

size_t block_workspace_bytes(int R);
int block_step_launch(float* W, int R, int64_t ldw, const float* U, int64_t ldu, int block,
                      int technique, int orders, float lam, float corr_damp, int metric, float* Err, int64_t ld_err,
                      float* Losses, unsigned char* codes, int64_t ld_codes, float* scales,
                      double* trace, void* workspace, size_t workspace_bytes, cudaStream_t st, bool reset_tickets = true);

constexpr int kStaticMaxRows = CRB_STATIC_MAX_ROWS;
// fixed tables of the block step (< 1 MiB) + per row 512 bytes of metric values, 512 bytes of
// sorted values, 128 bytes of sorted column indices and 256 bytes of selection lists
constexpr size_t kStaticScratchBytes = (size_t(1) << 20) + size_t(kStaticMaxRows) * 1408;

// The scratch itself.  In host code this name is only a handle for the runtime, not a device
// address: the address used at launch comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::mutex g_setup_mutex;
static void* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device, resolved once per device.
static int static_scratch_address(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return CRB_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return CRB_ERR_LAUNCH;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return CRB_OK;
}

}  // namespace crb

using namespace crb;

extern "C" {

int crb_block_step_static_max_rows(void) { return kStaticMaxRows; }

int crb_block_step_static(float* W, int R, int64_t ldw, const float* U, int64_t ldu, int block,
                          int technique, int orders, float lam, float corr_damp, int metric, float* Err,
                          float* Losses, uint8_t* codes, float* scales, double* trace,
                          unsigned* flags_out, void* stream) {
    if (R <= 0) return CRB_ERR_BAD_ARG;
    if (R > kStaticMaxRows || block_workspace_bytes(R) > kStaticScratchBytes) return CRB_ERR_STATIC_LIMIT;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != CRB_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the status word is the first thing in the scratch; it must describe this call only
    if (cudaMemsetAsync(scratch, 0, 64, st) != cudaSuccess) return CRB_ERR_LAUNCH;
    uint8_t* codes_base = codes ? codes - (int64_t)block * kBlock : nullptr;   // codes is [R, 128]
    rc = block_step_launch(W, R, ldw, U, ldu, block, technique, orders, lam, corr_damp, metric, Err, kBlock, Losses,
                           codes_base, kBlock, scales, trace, scratch, kStaticScratchBytes, st);
    if (rc != CRB_OK) return rc;
    if (flags_out &&
        cudaMemcpyAsync(flags_out, scratch, sizeof(unsigned), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return CRB_ERR_LAUNCH;
    return CRB_OK;
}

}  // extern "C"
