// Hessian accumulation  S += X^T X  on the 5th-generation tensor cores (tcgen05 + TMEM),
// operands staged by TMA.  Replaces BRAGPTQ.add_batch (bigptq.py:37-54).
//
// X is [T, C] row-major (channel contiguous), so both MMA operands are "MN-major": a TMA box
// of 64 channels x 64 tokens with 128-byte swizzle lands in shared memory as 8-token x 128-byte
// swizzle atoms, which is the canonical MN-major SWIZZLE_128B operand layout of tcgen05.mma
// (leading-dimension offset = one 64-channel box, stride offset = 1024 bytes per 8 tokens).
//
// Clusters of two CTAs (one per SM) walk the upper-triangle 256 x 256 output tiles persistently;
// a pair computes its tile with tcgen05.mma.cta_group::2 (M = 256 across the two SMs, N = 256).
// Warp roles per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (leader CTA only; owns the TMEM
// allocation), warps 2..9 = epilogue (two warps per TMEM lane quarter, one per column half).
// Two 256-column TMEM accumulators alternate.  The token dimension is cut into chunks; each
// chunk is accumulated in TMEM and then folded into float32 REGISTER accumulators by the CUDA
// cores (round to nearest), which bounds the length of any tensor-core running sum (its adder
// truncates) without touching memory; S is read-modified-written once per tile and call.
//
// float32 X (the single-linear configuration) is split by a pre-pass into two fp16 planes
// x*s = hi + lo (s a power of two); the tile then accumulates hi^T hi + hi^T lo + lo^T hi,
// which carries 22 significand bits of every product.
//
// Every mbarrier wait is bounded; on expiry the kernel raises CRB_FLAG_WAIT_LIMIT, all roles
// leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>
#include <stdlib.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "umma.cuh"

namespace crb {

constexpr int HT_M = 128;              // output rows per CTA (UMMA M = 256 over the pair)
constexpr int HT_N = 256;              // output columns per tile (UMMA N)
constexpr int HT_K = 64;               // tokens per pipeline stage
constexpr int HT_BOX = 64;             // channels per TMA box (128 bytes of 16-bit elements)
constexpr int HT_BOX_BYTES = HT_BOX * HT_K * 2;                          // 8 KiB
constexpr int HT_THREADS = 320;          // TMA warp, MMA warp, eight epilogue warps

// Shared-memory matrix descriptor of an MN-major, 128-byte-swizzled operand:
//   bits 0-13 start address >> 4, 16-29 leading-dimension byte offset >> 4 (between 64-element
//   boxes along M/N), 32-45 stride byte offset >> 4 (between 8-token groups), 46-47 version 1,
//   61-63 layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t mn_sw128_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D = f32, A/B = f16 (0) or bf16 (1), both MN-major.
__host__ __device__ constexpr uint32_t f16_idesc(int ab_format, int M, int N) {
    return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | (1u << 15) | (1u << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

struct HessArgs {
    float* S;            // [C, C] accumulator (upper-triangle tiles are updated)
    const float* inv_scale2;   // device scalar multiplying every accumulator (NULL = 1)
    unsigned* status;
    int C;
    int64_t T;
    int chunk_tokens;    // tokens accumulated in TMEM before they are added to S
    int n_pass;          // 1: X^T X from plane 0;  3: hi^T hi + hi^T lo + lo^T hi
    int ab_format;       // 0 f16, 1 bf16
    int n_tiles, n_col_tiles;
};

// ---------------------------------------------------------------------------------------------
// A cluster of two CTAs (two SMs) computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  CTA r of the pair loads the operand rows r*128..r*128+127 of the M
// side and of the N side, so every CTA stages 256 channel rows per 256 x 256 x K of work (a
// single CTA on a 128 x 256 tile would stage 384 per half the work): the L2 -> shared-memory
// traffic per flop is what limits this kernel.  The leader (cluster rank 0) issues all MMAs; both
// CTAs' TMA copies report to the leader's "full" barrier; MMA completion is committed to the
// barriers of both CTAs (two plain commits); each CTA drains its own 128 accumulator rows.
// ---------------------------------------------------------------------------------------------
constexpr int H2_STAGES = 6;
constexpr int H2_HALF_BYTES = 2 * HT_BOX_BYTES;                 // 128 channels x 64 tokens = 16 KiB
constexpr int H2_STAGE_BYTES = 2 * H2_HALF_BYTES;               // A half + B half = 32 KiB per CTA
constexpr int H2_SMEM = H2_STAGES * H2_STAGE_BYTES + 1024 + 256;
constexpr int H2_TILE = 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load of one CTA of a pair; the completion bytes go to `cluster_bar`, which may live in the peer.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)acc) : "memory");
}
// Arrives on `cluster_bar` (any CTA of the cluster) once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

// Linear index over the upper-triangle 256 x 256 tiles.  Tile rows are grouped in bands of
// H2_BAND; inside a band the index runs down each tile column before moving to the next one.
// The pairs work on consecutive indices at the same time and march through the tokens
// together, so a wave of 74 tiles covers about 8 x 9 tiles and reads ~17 distinct 256-channel
// slabs of X per token step through L2 instead of the ~66 a row-by-row order touches.
constexpr int H2_BAND = 8;
__device__ __forceinline__ void pair_tile_coords(int t, int nt, int* mi, int* nj) {
    int r0 = 0;
    for (;;) {
        const int h = min(H2_BAND, nt - r0);
        const int tri = h * (h + 1) / 2;
        const int band = tri + h * (nt - r0 - h);
        if (t < band) {
            if (t < tri) {
                int c = 0;
                while (t > c) { t -= c + 1; ++c; }       // column c of the triangle holds rows 0..c
                *mi = r0 + t; *nj = r0 + c;
            } else {
                t -= tri;
                *mi = r0 + t % h; *nj = r0 + h + t / h;
            }
            return;
        }
        t -= band;
        r0 += h;
    }
}

__global__ void __launch_bounds__(HT_THREADS, 1)
k_hessian_umma_pair(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                    const HessArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + H2_STAGES * H2_STAGE_BYTES);
    // bars[0..S) full (used in the leader), [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty (leader)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * H2_STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * H2_STAGES;
    const uint32_t tfull0 = empty0 + 8 * H2_STAGES, tempty0 = tfull0 + 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < H2_STAGES; ++s) { mbar_init(full0 + 8 * s, 2); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 16); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // the peer's barriers exist before anything remote touches them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_chunks = (int)((args.T + args.chunk_tokens - 1) / args.chunk_tokens);
    const int pairs = gridDim.x >> 1;
    const int pair = (int)cluster_id_x();
    const int nt = args.n_col_tiles;          // 256-wide tiles per dimension

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs): own 128 rows of the M side and of the N side ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = pair; t < args.n_tiles && ok; t += pairs) {
                int mi, nj;
                pair_tile_coords(t, nt, &mi, &nj);
                const int ca = mi * H2_TILE + (int)rank * 128, cb = nj * H2_TILE + (int)rank * 128;
                for (int ch = 0; ch < n_chunks && ok; ++ch) {
                    const int64_t t0 = (int64_t)ch * args.chunk_tokens;
                    const int64_t t1 = min(args.T, t0 + args.chunk_tokens);
                    for (int p = 0; p < args.n_pass && ok; ++p) {
                        const CUtensorMap* ma = (p == 2) ? &map1 : &map0;
                        const CUtensorMap* mb = (p == 1) ? &map1 : &map0;
                        for (int64_t tk = t0; tk < t1; tk += HT_K) {
                            ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag);
                            if (!ok) break;
                            const uint32_t sa = smem_u32(smem + stage * H2_STAGE_BYTES);
                            const uint32_t sb = sa + H2_HALF_BYTES;
                            const uint32_t fb = map_to_cta(full0 + 8 * stage, 0);      // the leader's barrier
                            mbar_expect_tx_cluster(fb, H2_STAGE_BYTES);
#pragma unroll
                            for (int b = 0; b < 2; ++b) {
                                tma_load_2d_pair(sa + b * HT_BOX_BYTES, ma, ca + b * HT_BOX, (int)tk, fb);
                                tma_load_2d_pair(sb + b * HT_BOX_BYTES, mb, cb + b * HT_BOX, (int)tk, fb);
                            }
                            if (++stage == H2_STAGES) { stage = 0; phase ^= 1; }
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the leader CTA only ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = f16_idesc(args.ab_format, 2 * HT_M, HT_N);
            uint32_t stage = 0, phase = 0, unit = 0;
            bool ok = true;
            for (int t = pair; t < args.n_tiles && ok; t += pairs) {
                for (int ch = 0; ch < n_chunks && ok; ++ch, ++unit) {
                    const uint32_t buf = unit & 1, use = unit >> 1;
                    ok = mbar_wait(tempty0 + 8 * buf, (use & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * HT_N;
                    const int64_t t0 = (int64_t)ch * args.chunk_tokens;
                    const int64_t t1 = min(args.T, t0 + args.chunk_tokens);
                    bool first = true;
                    for (int p = 0; p < args.n_pass && ok; ++p) {
                        for (int64_t tk = t0; tk < t1; tk += HT_K) {
                            ok = mbar_wait(full0 + 8 * stage, phase, abort_flag);
                            if (!ok) break;
                            tc_fence_after();
                            const uint32_t sa = smem_u32(smem + stage * H2_STAGE_BYTES);
                            const uint32_t sb = sa + H2_HALF_BYTES;
#pragma unroll
                            for (int k = 0; k < HT_K / 16; ++k) {
                                const uint64_t da = mn_sw128_desc(sa + k * 2048, HT_BOX_BYTES, 1024);
                                const uint64_t db = mn_sw128_desc(sb + k * 2048, HT_BOX_BYTES, 1024);
                                umma_f16_pair(d_tmem, da, db, idesc, !first);
                                first = false;
                            }
                            umma_commit_pair(empty0 + 8 * stage);                       // frees the stage here ...
                            umma_commit_pair(map_to_cta(empty0 + 8 * stage, 1));        // ... and in the peer
                            if (++stage == H2_STAGES) { stage = 0; phase ^= 1; }
                        }
                    }
                    if (ok) {
                        umma_commit_pair(tfull0 + 8 * buf);
                        umma_commit_pair(map_to_cta(tfull0 + 8 * buf, 1));
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): own 128 accumulator rows, all 256 columns.
        // Each token chunk's TMEM accumulator is folded into float32 registers (round to nearest);
        // S is read and written once per tile, after the last chunk. ----------------
        const int q = warp & 3;
        const int c_begin = ((warp - 2) >> 2) * (HT_N / 2);
        const float scale = args.inv_scale2 ? *args.inv_scale2 : 1.0f;
        const uint32_t tempty_leader = map_to_cta(tempty0, 0);
        uint32_t unit = 0;
        bool ok = true;
        for (int t = pair; t < args.n_tiles && ok; t += pairs) {
            int mi, nj;
            pair_tile_coords(t, nt, &mi, &nj);
            const int row = mi * H2_TILE + (int)rank * 128 + q * 32 + lane;
            float acc[4][32];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[u][j] = 0.f;
            for (int ch = 0; ch < n_chunks && ok; ++ch, ++unit) {
                const uint32_t buf = unit & 1, use = unit >> 1;
                ok = mbar_wait(tfull0 + 8 * buf, use & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * HT_N + c_begin;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float v[32];
                    tmem_ld32(taddr + 32 * u, v);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[u][j] += v[j];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * buf);
            }
            if (!ok) break;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int col = nj * H2_TILE + c_begin + 32 * u;
                // only columns at or right of this row's diagonal are ever read back
                if (row < args.C && col < args.C && col + 31 >= row) {
                    float4* dst = reinterpret_cast<float4*>(args.S + (int64_t)row * args.C + col);
                    float4 o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = dst[j];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        o[j].x = fmaf(acc[u][4 * j + 0], scale, o[j].x); o[j].y = fmaf(acc[u][4 * j + 1], scale, o[j].y);
                        o[j].z = fmaf(acc[u][4 * j + 2], scale, o[j].z); o[j].w = fmaf(acc[u][4 * j + 3], scale, o[j].w);
                        dst[j] = o[j];
                    }
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: report it and give copies that may still be in flight 2 ms to land
        if (threadIdx.x == 0) atomicOr(args.status, CRB_FLAG_WAIT_LIMIT);
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) { }
    }
    cluster_sync_all();                       // neither CTA leaves while the peer may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---- float32 input: amax, then split into two fp16 planes ------------------------------------
__global__ void k_amax(const float* __restrict__ X, int64_t T, int C, int64_t ldx, unsigned* amax_bits) {
    float m = 0.f;
    const int64_t n = T * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = fabsf(X[(i / C) * ldx + (i % C)]);
        m = fmaxf(m, isfinite(v) ? v : 0.f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));
}

// scale s = 2^e with amax * s in [2^13, 2^14); planes hi = fp16(x s), lo = fp16(x s - hi).
__global__ void k_split_f32(const float* __restrict__ X, int64_t T, int C, int64_t ldx,
                            const unsigned* __restrict__ amax_bits, __half* __restrict__ hi,
                            __half* __restrict__ lo, float* __restrict__ inv_scale2) {
    const float amax = __uint_as_float(*amax_bits);
    int e = 0;
    if (amax > 0.f) { int ex; frexpf(amax, &ex); e = 14 - ex; }     // amax = f * 2^ex, f in [0.5, 1)
    e = max(-60, min(60, e));
    const float s = ldexpf(1.0f, e);
    if (blockIdx.x == 0 && threadIdx.x == 0) *inv_scale2 = ldexpf(1.0f, -2 * e);
    const int64_t n = T * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = X[(i / C) * ldx + (i % C)] * s;
        const __half h = __float2half_rn(v);
        hi[i] = h;
        lo[i] = __float2half_rn(v - __half2float(h));
    }
}

// H = scale * S on and above the diagonal, mirrored below it.
__global__ void k_hessian_finalize(float* __restrict__ S, int C, float scale) {
    __shared__ float tile[32][33];
    const int bi = blockIdx.y, bj = blockIdx.x;
    if (bj < bi) return;
    const int tx = threadIdx.x, ty = threadIdx.y;            // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const int i = bi * 32 + r, j = bj * 32 + tx;
        float v = 0.f;
        if (i < C && j < C) {
            v = S[(int64_t)i * C + j] * scale;
            if (j >= i) S[(int64_t)i * C + j] = v;
        }
        tile[r][tx] = v;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int i = bj * 32 + r, j = bi * 32 + tx;         // transposed position
        if (i < C && j < C && j < i) S[(int64_t)i * C + j] = tile[tx][r];
    }
}

// Number of floats in front of row r in the packed form: rows of band b = r / 256 keep their
// columns from 256 b on (the accumulation kernel only maintains those tiles).
__host__ __device__ inline long long packed_row_offset(int r, int C) {
    const long long b = r / H2_TILE, in_band = r % H2_TILE;
    // full bands in front: sum_{k < b} 256 * (C - 256 k)
    return (long long)H2_TILE * (b * C - (long long)H2_TILE * b * (b - 1) / 2) + in_band * ((long long)C - H2_TILE * b);
}

// Copies the maintained part of S (its upper-triangle 256 x 256 tiles) into a contiguous buffer or
// back, so that a sum over ranks moves half the bytes.  One CTA per row.
__global__ void __launch_bounds__(256)
k_hessian_pack(float* __restrict__ S, int C, float* __restrict__ packed, int unpack) {
    const int r = blockIdx.x;
    const int c0 = r / H2_TILE * H2_TILE;
    float* row = S + (int64_t)r * C + c0;
    float* dst = packed + packed_row_offset(r, C);
    const int n4 = (C - c0) >> 2;                               // C and c0 are multiples of 128
    float4* a = reinterpret_cast<float4*>(row);
    float4* b = reinterpret_cast<float4*>(dst);
    for (int k = threadIdx.x; k < n4; k += blockDim.x) {
        if (unpack) a[k] = b[k]; else b[k] = a[k];
    }
}

// ---- host side ----------------------------------------------------------------------------------
static int make_map(CUtensorMap* map, const void* base, int dtype, int64_t T, int C, int64_t ld) {
    const CUtensorMapDataType dt = (dtype == CRB_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return make_tensor_map_2d(map, base, dt, 2, (uint64_t)C, (uint64_t)T, (uint64_t)ld, HT_BOX, HT_K);
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Tokens accumulated on the tensor cores before the running sum is folded into S by float32
// adds (a multiple of the 64-token stage).
constexpr int kHessianChunkTokens = 2048;

size_t hessian_workspace_bytes(int C, int64_t T, int dtype) {
    size_t b = 256;                                           // amax + inv_scale2 + status
    if (dtype == CRB_F32) b += 2 * align256((size_t)T * C * sizeof(__half));
    return b;
}

int hessian_accumulate_launch(const void* X, int dtype, int64_t T, int C, int64_t ldx, float* S,
                              void* workspace, size_t workspace_bytes, cudaStream_t st) {
    if (!X || !S || !workspace || T <= 0 || C <= 0 || ldx < C) return CRB_ERR_BAD_ARG;
    if (C % kBlock) return CRB_ERR_UNSUPPORTED;
    if (dtype != CRB_F32 && dtype != CRB_F16 && dtype != CRB_BF16) return CRB_ERR_BAD_ARG;
    if (T >= (1ll << 31)) return CRB_ERR_UNSUPPORTED;
    if (workspace_bytes < hessian_workspace_bytes(C, T, dtype)) return CRB_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(S) & 15) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255))
        return CRB_ERR_BAD_ARG;
    unsigned* status = static_cast<unsigned*>(workspace);          // word 0: sticky status flags
    unsigned* amax = status + 1;
    float* inv_scale2 = reinterpret_cast<float*>(status + 2);

    CUtensorMap map0, map1;
    HessArgs a;
    a.S = S; a.status = status; a.C = C; a.T = T;
    a.chunk_tokens = kHessianChunkTokens;
    a.n_col_tiles = (C + H2_TILE - 1) / H2_TILE;
    a.n_tiles = a.n_col_tiles * (a.n_col_tiles + 1) / 2;
    if (dtype == CRB_F32) {
        if (ldx & 3) return CRB_ERR_BAD_ARG;
        __half* hi = reinterpret_cast<__half*>(static_cast<char*>(workspace) + 256);
        __half* lo = reinterpret_cast<__half*>(static_cast<char*>(workspace) + 256 + align256((size_t)T * C * sizeof(__half)));
        if (cudaMemsetAsync(amax, 0, 8, st) != cudaSuccess) return CRB_ERR_LAUNCH;
        k_amax<<<296, 256, 0, st>>>(static_cast<const float*>(X), T, C, ldx, amax);
        CRB_LAUNCHED();
        k_split_f32<<<592, 256, 0, st>>>(static_cast<const float*>(X), T, C, ldx, amax, hi, lo, inv_scale2);
        CRB_LAUNCHED();
        int rc = make_map(&map0, hi, CRB_F16, T, C, C);
        if (rc == CRB_OK) rc = make_map(&map1, lo, CRB_F16, T, C, C);
        if (rc != CRB_OK) return rc;
        a.n_pass = 3; a.ab_format = 0; a.inv_scale2 = inv_scale2;
    } else {
        if (ldx & 7) return CRB_ERR_BAD_ARG;
        int rc = make_map(&map0, X, dtype, T, C, ldx);
        if (rc != CRB_OK) return rc;
        map1 = map0;
        a.n_pass = 1; a.ab_format = (dtype == CRB_BF16) ? 1 : 0; a.inv_scale2 = nullptr;
    }
    static PerDeviceSetup once;
    int sms = 148;
    const int rc_setup = once.run([] {
        return cudaFuncSetAttribute(k_hessian_umma_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, H2_SMEM) == cudaSuccess
                   ? (int)CRB_OK : (int)CRB_ERR_LAUNCH;
    }, &sms);
    if (rc_setup != CRB_OK) return rc_setup;
    // clusters of two CTAs over the 256 x 256 upper-triangle tiles
    const int pairs = a.n_tiles < sms / 2 ? a.n_tiles : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(HT_THREADS);
    cfg.dynamicSmemBytes = H2_SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, k_hessian_umma_pair, map0, map1, a) != cudaSuccess) return CRB_ERR_LAUNCH;
    CRB_LAUNCHED();
    return CRB_OK;
}

long long hessian_packed_floats(int C) { return C > 0 ? packed_row_offset(C, C) : 0; }

int hessian_pack_launch(float* S, int C, float* packed, int unpack, cudaStream_t st) {
    if (!S || !packed || C <= 0 || (C % kBlock)) return CRB_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(S) | reinterpret_cast<uintptr_t>(packed)) & 15) return CRB_ERR_BAD_ARG;
    k_hessian_pack<<<C, 256, 0, st>>>(S, C, packed, unpack);
    CRB_LAUNCHED();
    return CRB_OK;
}

int hessian_finalize_launch(float* S, int C, float scale, cudaStream_t st) {
    if (!S || C <= 0) return CRB_ERR_BAD_ARG;
    const int nb = (C + 31) / 32;
    k_hessian_finalize<<<dim3(nb, nb), dim3(32, 8), 0, st>>>(S, C, scale);
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
