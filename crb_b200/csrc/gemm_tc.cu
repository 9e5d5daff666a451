// float32-faithful GEMM on the tensor cores:  C = alpha * A * op(B) + beta * C,  all float32.
//
// The reference multiplies in full float32 (TF32 is switched off, bigptq.py:11-12), so a plain
// TF32 product (10-bit mantissa) would not do.  Every operand tile x is taken as hi + lo with
// hi = x with the low 13 mantissa bits cleared (exactly a TF32 number) and lo = x - hi (exact in
// float32), and three tcgen05.mma kind::tf32 products hi*hi + hi*lo + lo*hi are accumulated:
// 21-22 significand bits per product.  The tensor core reads only the upper 19 bits of a TF32
// operand, so the raw float32 tile as TMA delivered it IS the hi plane; the splitter warps only
// write the lo plane next to it (the accuracy test of the GEMM pins this behaviour: a part that
// rounded instead of truncating would fail it at the 1e-3 level).  The kernel is bound by
// shared-memory bandwidth (every MMA re-reads its 4-byte operands), not by the MMA rate.
//
// Used by the trailing update W[:, i2:] -= Err @ U[i1:i2, i2:] (bigptq.py:264) and by the
// panel / rank-128 / inverse-merge products of the blocked factorisation.
//
// One persistent CTA per SM over 128 x 256 output tiles, four warpgroups: warp 0 TMA producer
// (float32 tiles, 64-byte swizzle), warp 1 MMA issuer (owns TMEM), warps 4-7 write the lo plane
// of the landed tiles, warps 8-15 epilogue.  Four shared-memory stages of K = 16, two 256-column
// TMEM accumulators.
//
// The tensor core truncates (rounds toward zero) every time it adds to its float32 accumulator,
// a bias that grows with the length of the chain (measured on a 4096 x 4096 factorisation with
// condition number 6e4: chains of K = 1024 gave a factor 7 x less accurate than the float32
// library chain, K = 128 chains 5 x its error on the diagonal, K = 32 chains parity).  The MMAs
// therefore accumulate two shared-memory stages (K = 32, 12 instructions) in TMEM; the epilogue
// warps fold every such chunk into float32 REGISTER accumulators with round-to-nearest adds while
// the next chunk runs in the other TMEM buffer, and write C once per tile.  The epilogue warpgroups hold 128 accumulator registers per
// thread; setmaxnreg moves registers to them from the producer / splitter warpgroups.
// A is [M, K] row-major
// (K-major operand); B is [N, K] row-major (K-major) or [K, N] row-major (MN-major operand).
// All mbarrier waits are bounded (2 s); on expiry CRB_FLAG_WAIT_LIMIT is raised and the kernel
// drains and returns.
#include "common.cuh"
#include "umma.cuh"

namespace crb {

// K per shared-memory stage: 32 (128-byte rows, 2 stages) or 16 (64-byte rows, 4 stages: the
// deeper ring hides the TMA latency between "MMAs retired" and "next tile split").
constexpr int GT_M = 128, GT_N = 256, GT_K = 16;
static_assert(GT_K == 32 || GT_K == 16, "stage depth");
constexpr int GT_STAGES = GT_K == 32 ? 2 : 4;
constexpr int GT_A_BYTES = GT_M * GT_K * 4;                 // 16 / 8 KiB
constexpr int GT_B_BYTES = GT_N * GT_K * 4;                 // 32 / 16 KiB
constexpr int GT_RAW_BYTES = GT_A_BYTES + GT_B_BYTES;       // hi planes (TMA destination)
constexpr int GT_STAGE_BYTES = 2 * GT_RAW_BYTES;            // + lo planes
constexpr int GT_BOX_BYTES = 32 * GT_K * 4;                 // MN-major B: one box of 32 columns x GT_K k-rows
constexpr int GT_EPI_BYTES = 8 * 32 * 33 * 4;                 // per-warp transpose patches of the epilogue
constexpr int GT_SMEM = GT_STAGES * GT_STAGE_BYTES + 256 + GT_EPI_BYTES + 1024;
constexpr int GT_THREADS = 512;              // warpgroups: TMA + MMA (+ 2 idle warps), 4 splitter warps, 2 x 4 epilogue warps
constexpr int GT_CHUNK_STEPS = 32 / GT_K;     // stages accumulated in TMEM (K = 32) before the fold into registers
// registers per thread after the reallocation; the sum over the four warpgroups is 512 = 4 x 128
constexpr int GT_REGS_IO = 56, GT_REGS_SPLIT = 72, GT_REGS_EPI = 192;
static_assert(GT_REGS_IO + GT_REGS_SPLIT + 2 * GT_REGS_EPI <= 4 * 128, "register budget of a CTA");

struct GemmArgs {
    float* C;
    int64_t ldc;
    int M, N, K;
    float alpha, beta;
    int b_is_nk;          // 1: B is [N, K] row-major (K-major operand); 0: B is [K, N] row-major (MN-major)
    int lower_only;       // write only 128 x 128 blocks on or below the diagonal (tiles above it are skipped)
    int b_slabs;          // MN-major B: 1 = one 3-D copy per stage (map_b is a slab map), 0 = eight 2-D copies
    int tri;              // bit 0: op(B)[k][n] = 0 for k < n (lower-triangular [K, N] operand): K starts at the tile's column
                          // bit 1: A[m][k] = 0 for k > m (lower-triangular A): K ends with the tile's last row
    int m_tiles, n_tiles;
    unsigned* status;
    unsigned long long wait_ns;   // limit of every barrier wait
    int withhold_loads;   // self-test only: the producer issues nothing, so the first wait runs out
};

// K-major operand: rows of GT_K floats (128 bytes with the 128-byte swizzle, 64 bytes with the
// 64-byte swizzle), 8-row groups 8 rows apart.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fffu);
    d |= (uint64_t)1 << 16;                               // leading offset: unused for swizzled K-major
    d |= (uint64_t)((8 * GT_K * 4) >> 4) << 32;           // stride between 8-row groups
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(GT_K == 32 ? 2 : 4) << 61;            // SWIZZLE_128B / SWIZZLE_64B
    return d;
}
// MN-major 32-bit operand: the only shared-memory layout the tensor core accepts is the 128-byte
// swizzle with 32-byte atoms (layout type 1; TMA mode SWIZZLE_128B_ATOM_32B): rows of 128 bytes
// (32 columns), swizzle period 4 k-rows (512 bytes).  Boxes of 32 columns x 32 k-rows (4 KiB) sit
// side by side: leading offset = one box, stride offset = 512 bytes between 4-row k groups.
__device__ __forceinline__ uint64_t mnmajor_sw128_desc(uint32_t saddr, uint32_t box_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fffu);
    d |= (uint64_t)((box_bytes >> 4) & 0x3fffu) << 16;    // between 32-column boxes
    d |= (uint64_t)(512 >> 4) << 32;                      // between 4-row k groups
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;                               // SWIZZLE_128B_BASE32B
    return d;
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)acc) : "memory");
}
// kind::tf32: D = f32 (1 << 4), A and B formats TF32 (2), A K-major, B major per call.
__device__ __forceinline__ uint32_t tf32_idesc(int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(GT_N >> 3) << 17) | ((uint32_t)(GT_M >> 4) << 24);
}

__device__ __forceinline__ bool tile_skipped(const GemmArgs& g, int mi, int nj) {
    return g.lower_only && (nj * GT_N > mi * GT_M + GT_M - 1);
}

// K steps [k0, k1) a tile has to run: all of them, less the part a triangular operand makes zero.
__device__ __forceinline__ void tile_k_range(const GemmArgs& g, int mi, int nj, int* k0, int* k1) {
    int lo = 0, hi = g.K / GT_K;
    if (g.tri & 1) lo = (nj * GT_N) / GT_K;
    if (g.tri & 2) hi = min(hi, (mi * GT_M + GT_M + GT_K - 1) / GT_K);
    *k0 = min(lo, hi - 1);
    *k1 = hi;
}

__global__ void __launch_bounds__(GT_THREADS, 1)
k_gemm_tf32x3(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GT_STAGES * GT_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * GT_STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars);                 // TMA landed          (count 1 + tx)
    const uint32_t ready0 = full0 + 8 * GT_STAGES;         // hi / lo split done  (count 4 warps)
    const uint32_t empty0 = ready0 + 8 * GT_STAGES;        // MMAs retired        (count 1)
    const uint32_t tfull0 = empty0 + 8 * GT_STAGES, tempty0 = tfull0 + 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GT_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1); mbar_init(ready0 + 8 * s, 4); mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    chain_wait();          // operands and C belong to the kernels in front of this one in the stream
    const uint32_t tmem_base = *tmem_slot;
    const int total = g.m_tiles * g.n_tiles;
    // Each warpgroup first hands over / takes registers (uniform per warpgroup), then runs its role.
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(GT_REGS_IO));
    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, armed = 0, armed_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok && !g.withhold_loads; t += gridDim.x) {
                const int mi = t / g.n_tiles, nj = t % g.n_tiles;
                if (tile_skipped(g, mi, nj)) continue;
                int ks0, ks1;
                tile_k_range(g, mi, nj, &ks0, &ks1);
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, g.wait_ns);
                    if (!ok) break;
                    const uint32_t sa = smem_u32(smem + stage * GT_STAGE_BYTES);
                    const uint32_t sb = sa + GT_A_BYTES;
                    const uint32_t fb = full0 + 8 * stage;
                    mbar_expect_tx(fb, GT_RAW_BYTES);
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    tma_load_2d(sa, &map_a, ks * GT_K, mi * GT_M, fb);                    // 32 k x 128 rows
                    if (g.b_is_nk) {
                        tma_load_2d(sb, &map_b, ks * GT_K, nj * GT_N, fb);                // 32 k x 256 rows
                    } else if (g.b_slabs) {
                        tma_load_3d(sb, &map_b, 0, ks * GT_K, nj * (GT_N / 32), fb);      // 8 slabs of 32 cols x 32 k-rows
                    } else {
#pragma unroll
                        for (int b = 0; b < GT_N / 32; ++b)                               // 32 cols x 32 k-rows each
                            tma_load_2d(sb + b * GT_BOX_BYTES, &map_b, nj * GT_N + b * 32, ks * GT_K, fb);
                    }
                    if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            for (int s = 0; s < GT_STAGES; ++s) {          // drain copies in flight before smem goes away
                if (!(armed >> s & 1u)) continue;
                const unsigned long long t0 = global_ns();
                while (!mbar_try_wait(full0 + 8 * s, (armed_phase >> s) & 1u))
                    if (global_ns() - t0 > g.wait_ns) { *abort_flag = 1; break; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = tf32_idesc(g.b_is_nk ? 0 : 1);
            uint32_t stage = 0, phase = 0, unit = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int mi = t / g.n_tiles, nj = t % g.n_tiles;
                if (tile_skipped(g, mi, nj)) continue;
                int ks0, ks1;
                tile_k_range(g, mi, nj, &ks0, &ks1);
                for (int kc = ks0; kc < ks1 && ok; kc += GT_CHUNK_STEPS, ++unit) {
                    const uint32_t buf = unit & 1, use = unit >> 1;
                    ok = mbar_wait(tempty0 + 8 * buf, (use & 1) ^ 1, abort_flag, g.wait_ns);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * GT_N;
                    const int kc1 = min(kc + GT_CHUNK_STEPS, ks1);
                    bool first = true;
                    for (int ks = kc; ks < kc1; ++ks) {
                        ok = mbar_wait(ready0 + 8 * stage, phase, abort_flag, g.wait_ns);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t a_hi = smem_u32(smem + stage * GT_STAGE_BYTES), b_hi = a_hi + GT_A_BYTES;
                        const uint32_t a_lo = a_hi + GT_RAW_BYTES, b_lo = b_hi + GT_RAW_BYTES;
#pragma unroll
                        for (int k = 0; k < GT_K / 8; ++k) {
                            // one MMA consumes K = 8 float32: 32 bytes along a K-major row, or one
                            // 8-row group (1024 bytes) of an MN-major box
                            const uint32_t ao = k * 32, bo = g.b_is_nk ? k * 32 : k * 1024;
                            const uint64_t dah = kmajor_sw128_desc(a_hi + ao), dal = kmajor_sw128_desc(a_lo + ao);
                            const uint64_t dbh = g.b_is_nk ? kmajor_sw128_desc(b_hi + bo) : mnmajor_sw128_desc(b_hi + bo, GT_BOX_BYTES);
                            const uint64_t dbl = g.b_is_nk ? kmajor_sw128_desc(b_lo + bo) : mnmajor_sw128_desc(b_lo + bo, GT_BOX_BYTES);
                            umma_tf32(d_tmem, dal, dbh, idesc, !first);      // small terms first
                            umma_tf32(d_tmem, dah, dbl, idesc, true);
                            umma_tf32(d_tmem, dah, dbh, idesc, true);
                            first = false;
                        }
                        umma_commit(empty0 + 8 * stage);
                        if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
                    }
                    if (ok) umma_commit(tfull0 + 8 * buf);
                }
            }
        }
    }   // warps 2 and 3 only fill the first warpgroup
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(GT_REGS_SPLIT));
        // ---------------- splitter: lo = x - (x with 13 low mantissa bits cleared) ----------------
        const int ctid = threadIdx.x - 128;                 // 0..127
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            const int mi = t / g.n_tiles, nj = t % g.n_tiles;
            if (tile_skipped(g, mi, nj)) continue;
            int ks0, ks1;
            tile_k_range(g, mi, nj, &ks0, &ks1);
            for (int ks = ks0; ks < ks1; ++ks) {
                ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, g.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                float4* hi = reinterpret_cast<float4*>(smem + stage * GT_STAGE_BYTES);
                float4* lo = reinterpret_cast<float4*>(smem + stage * GT_STAGE_BYTES + GT_RAW_BYTES);
#pragma unroll 4
                for (int i = ctid; i < GT_RAW_BYTES / 16; i += 128) {
                    const float4 x = hi[i];
                    float4 h, l;
                    h.x = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u); l.x = x.x - h.x;
                    h.y = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u); l.y = x.y - h.y;
                    h.z = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u); l.z = x.z - h.z;
                    h.w = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u); l.w = x.w - h.w;
                    lo[i] = l;          // the raw tile itself serves as the hi plane (see the file header)
                }
                // make the generic-proxy writes visible to the tensor core (async proxy)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(ready0 + 8 * stage);
                if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(GT_REGS_EPI));
        // ---------------- epilogue: warps 8..15; warp w reads TMEM lanes 32 * (w % 4) .. +31 and the
        // column half (w - 8) / 4 of the accumulator ----------------
        const int q = warp & 3;
        const int c_begin = ((warp - 8) >> 2) * (GT_N / 2);
        uint32_t unit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            const int mi = t / g.n_tiles, nj = t % g.n_tiles;
            if (tile_skipped(g, mi, nj)) continue;
            int ks0, ks1;
            tile_k_range(g, mi, nj, &ks0, &ks1);
            // ---- fold the chunks of this tile into registers (thread = one accumulator row) ----
            float acc[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[c][j] = 0.f;
            for (int kc = ks0; kc < ks1 && ok; kc += GT_CHUNK_STEPS, ++unit) {
                const uint32_t buf = unit & 1, use = unit >> 1;
                ok = mbar_wait(tfull0 + 8 * buf, use & 1, abort_flag, g.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * GT_N + c_begin;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float v[32];
                    tmem_ld32(taddr + 32 * c, v);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[c][j] += v[j];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * buf);     // the MMAs may reuse this buffer
            }
            if (!ok) break;
            // ---- write the tile.  Every lane holds one row (32 columns per chunk): written like that,
            // each instruction would touch 32 different cache lines.  The 32 x 32 chunk is transposed
            // through a per-warp shared-memory patch instead, so that a warp instruction covers
            // 4 rows x 128 contiguous bytes.  Lane l then owns rows (l / 8) + 4k, k = 0..7, and
            // columns 4 (l % 8) .. +3 of the chunk. ----
            const int r_sub = lane >> 3, cg = lane & 7;
            const int row0 = mi * GT_M + q * 32 + r_sub;                 // + 4k
            const int colbase = nj * GT_N + c_begin + 4 * cg;            // + 32c
            auto live = [&](int c, int k) {
                const int row = row0 + 4 * k, col = colbase + 32 * c;
                // lower_only: nothing is written above the 128 x 128 block that holds the diagonal,
                // so that a triangular matrix updated this way keeps exact zeros there
                return row < g.M && col < g.N && !(g.lower_only && col > (row | 127));
            };
            // beta == 1 (the rank-k updates): C += alpha * acc goes out as vector reductions that
            // the L2 performs, so the SM never waits for the old values of C
            const bool use_red = (g.beta == 1.0f);
            float* patch = reinterpret_cast<float*>(smem + GT_STAGES * GT_STAGE_BYTES + 256) + (warp - 8) * (32 * 33);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int j = 0; j < 32; ++j) patch[lane * 33 + j] = acc[c][j];
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float* src = patch + (r_sub + 4 * k) * 33 + 4 * cg;
                    if (live(c, k)) {
                        float* dst = g.C + (int64_t)(row0 + 4 * k) * g.ldc + colbase + 32 * c;
                        if (use_red) {
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                         ::"l"(dst), "f"(g.alpha * src[0]), "f"(g.alpha * src[1]),
                                           "f"(g.alpha * src[2]), "f"(g.alpha * src[3]) : "memory");
                        } else {
                            float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (g.beta != 0.f) w = *reinterpret_cast<const float4*>(dst);
                            w.x = fmaf(g.alpha, src[0], g.beta * w.x);
                            w.y = fmaf(g.alpha, src[1], g.beta * w.y);
                            w.z = fmaf(g.alpha, src[2], g.beta * w.z);
                            w.w = fmaf(g.alpha, src[3], g.beta * w.w);
                            *reinterpret_cast<float4*>(dst) = w;
                        }
                    }
                }
                __syncwarp();
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && g.status) atomicOr(g.status, CRB_FLAG_WAIT_LIMIT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// C[M,N] = alpha * A[M,K] * op(B) + beta * C on the tensor cores.
// Requirements: K % 16 == 0, N % 32 == 0, leading dimensions % 4 == 0, 16-byte aligned bases.
// `status` (device, may be NULL) receives CRB_FLAG_WAIT_LIMIT if a bounded wait ran out.
// `max_ctas` > 0 caps the persistent grid (default: one CTA per SM).
// `shape` is a set of GEMM_* flags: GEMM_LOWER_ONLY writes only the 128 x 128 blocks on or below
// the diagonal of C; GEMM_B_LOWER / GEMM_A_LOWER promise a lower-triangular [K, N] operand B /
// [M, K] operand A, whose zero part is then not multiplied.
int gemm_tf32x3(bool b_is_nk, int shape, int M, int N, int K, float alpha, const float* A, int64_t lda,
                const float* B, int64_t ldb, float beta, float* C, int64_t ldc, unsigned* status,
                cudaStream_t st, const GemmSelfTest* selftest, int max_ctas) {
    if (M <= 0 || N <= 0) return CRB_OK;
    const bool lower_only = (shape & GEMM_LOWER_ONLY) != 0;
    if ((shape & GEMM_B_LOWER) && (b_is_nk || N > K)) return CRB_ERR_BAD_ARG;
    if ((shape & GEMM_A_LOWER) && M > K) return CRB_ERR_BAD_ARG;
    if (K <= 0 || (K % GT_K) || (N % 32) || (lda & 3) || (ldb & 3) || (ldc & 3)) return CRB_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return CRB_ERR_BAD_ARG;
    CUtensorMap map_a, map_b;
    const CUtensorMapSwizzle ksw = GT_K == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    int rc = make_tensor_map_2d(&map_a, A, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)K, (uint64_t)M, (uint64_t)lda,
                                GT_K, GT_M, ksw);
    if (rc != CRB_OK) return rc;
    if (b_is_nk)
        rc = make_tensor_map_2d(&map_b, B, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)K, (uint64_t)N, (uint64_t)ldb,
                                GT_K, GT_N, ksw);
    int b_slabs = 0;
    if (!b_is_nk) {
        // one 3-D copy for the eight 32-column slabs of a stage when the driver accepts that shape
        rc = make_tensor_map_slabs(&map_b, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, GT_K, GT_N / 32,
                                   CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        if (rc == CRB_OK) {
            b_slabs = 1;
        } else {
            rc = make_tensor_map_2d(&map_b, B, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)N, (uint64_t)K, (uint64_t)ldb,
                                    32, GT_K, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        }
    }
    if (rc != CRB_OK) return rc;
    GemmArgs g;
    g.b_slabs = b_slabs;
    g.C = C; g.ldc = ldc; g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.beta = beta;
    g.b_is_nk = b_is_nk ? 1 : 0; g.lower_only = lower_only ? 1 : 0;
    g.tri = ((shape & GEMM_B_LOWER) ? 1 : 0) | ((shape & GEMM_A_LOWER) ? 2 : 0);
    g.m_tiles = (M + GT_M - 1) / GT_M; g.n_tiles = (N + GT_N - 1) / GT_N;
    g.status = status;
    g.wait_ns = selftest ? selftest->wait_ns : kWaitLimitNs;
    g.withhold_loads = selftest ? selftest->withhold_loads : 0;
    static PerDeviceSetup once;
    int sms = 148;
    const int rc_setup = once.run([] {
        if (cudaFuncSetAttribute(k_gemm_tf32x3, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM) != cudaSuccess)
            return (int)CRB_ERR_LAUNCH;
        // The register reallocation inside the kernel can only hand out what the CTA was launched
        // with: refuse to launch a build whose register file share is smaller than the plan needs
        // (an epilogue warpgroup would wait for registers that never become free).
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, k_gemm_tf32x3) != cudaSuccess) return (int)CRB_ERR_LAUNCH;
        if (fa.numRegs * GT_THREADS < (GT_REGS_IO + GT_REGS_SPLIT + 2 * GT_REGS_EPI) * 128) return (int)CRB_ERR_UNSUPPORTED;
        return (int)CRB_OK;
    }, &sms);
    if (rc_setup != CRB_OK) return rc_setup;
    const int total = g.m_tiles * g.n_tiles;
    int ctas = total < sms ? total : sms;
    if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;     // leave SMs to whatever runs beside this product
    launch_chained(k_gemm_tf32x3, ctas, GT_THREADS, GT_SMEM, st, map_a, map_b, g);
    CRB_LAUNCHED();
    return CRB_OK;
}


}  // namespace crb
