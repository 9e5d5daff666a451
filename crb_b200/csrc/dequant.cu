// Rebuilds the float32 weights of a binarized linear from its packed form: sign planes, the
// low / mid group plane, the salient columns of every 128-column block and the per-row scales.
//
// The reference keeps only the de-quantized weights (bigptq.py:276-280) and its --save is commented
// out (run.py:1033-1039); this is the format that makes the result storable at about two bits per
// weight plus scales, and the kernel that turns it back into exactly the numbers the block step
// wrote (same float32 expressions, same rounding: see group_order1 / group_order2 in block_step.cu).
//
// Layout (R rows, C columns, nblk = C / 128 blocks):
//   b1      [R, C/8]        bit (r, c) = first sign of the element is +1 (else -1)
//   lm      [R, C/8]        bit (r, c) = element belongs to the "mid" group (else "low"); unused at salient columns
//   salcol  [C]             position of the column inside its block's salient set, 255 = not salient
//   b2      per block b: [R, pitch_b] bytes at b2_off[b], pitch_b = ceil(n_salient_b / 8);
//           bit (r, k) = second sign of the k-th salient column is +1
//   scales  [nblk, R, 8]    low (mean, alpha), mid (mean, alpha), salient (4 values, per technique)
// Elements whose sign is 0 (a centred value of exactly 0) or that belong to no group are not
// representable in a bit plane; the packer lists them with their values and the caller patches
// them after this kernel.
#include "common.cuh"

namespace crb {

__global__ void __launch_bounds__(256)
k_dequantize(float* __restrict__ W, int R, int C, int64_t ldw, int technique,
             const unsigned char* __restrict__ b1, const unsigned char* __restrict__ lm,
             const unsigned char* __restrict__ salcol, const unsigned char* __restrict__ b2,
             const long long* __restrict__ b2_off, const int* __restrict__ b2_pitch,
             const float* __restrict__ scales) {
    // one warp per (row, block): lane l rebuilds columns 4 l .. 4 l + 3 of the block.  The grid is
    // (blocks, row groups of 8), so no index needs a division.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.y * 8 + warp, blk = blockIdx.x;
    if (row >= R) return;
    const int col = blk * kBlock + 4 * lane;
    const float* sc = scales + ((size_t)blk * R + row) * 8;
    const float4 s0 = *reinterpret_cast<const float4*>(sc), s1 = *reinterpret_cast<const float4*>(sc + 4);
    const size_t bit_base = (size_t)row * (C >> 3) + (col >> 3);
    const unsigned sh = (lane & 1) * 4;                       // this lane's four bits inside the byte
    const unsigned v1 = (unsigned)b1[bit_base] >> sh, vg = (unsigned)lm[bit_base] >> sh;
    const unsigned scol = *reinterpret_cast<const unsigned*>(salcol + col);      // four column entries
    const unsigned char* b2row = b2 + b2_off[blk] + (size_t)row * b2_pitch[blk];
    const bool braq = technique == CRB_TECH_BRAQ;
    float q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        // +1 / -1 from a bit: flip the sign bit of -1.0f
        const float B1 = __uint_as_float(0xbf800000u ^ (((v1 >> e) & 1u) << 31));
        const unsigned sk = (scol >> (8 * e)) & 255u;
        if (sk == 255u) {
            const bool mid = (vg >> e) & 1u;                  // else low
            q[e] = __fadd_rn((mid ? s0.w : s0.y) * B1, mid ? s0.z : s0.x);
        } else {
            const float B2 = __uint_as_float(0xbf800000u ^ ((((unsigned)b2row[sk >> 3] >> (sk & 7u)) & 1u) << 31));
            q[e] = braq ? __fadd_rn(__fadd_rn(s1.y * B1, s1.x), __fadd_rn(s1.w * B2, s1.z))
                        : __fadd_rn(__fadd_rn(s1.x, __fmul_rn(s1.y, B1)), __fmul_rn(s1.z, B2));
        }
    }
    *reinterpret_cast<float4*>(W + (int64_t)row * ldw + col) = make_float4(q[0], q[1], q[2], q[3]);
}

int dequantize_launch(float* W, int R, int C, int64_t ldw, int technique, const unsigned char* b1,
                      const unsigned char* lm, const unsigned char* salcol, const unsigned char* b2,
                      const long long* b2_off, const int* b2_pitch, const float* scales, cudaStream_t st) {
    if (!W || !b1 || !lm || !salcol || !b2 || !b2_off || !b2_pitch || !scales || R <= 0 || C <= 0) return CRB_ERR_BAD_ARG;
    if (C % kBlock) return CRB_ERR_UNSUPPORTED;
    if (technique < CRB_TECH_BRAQ || technique > CRB_TECH_CRB_SYMDAMP_NOREFINE) return CRB_ERR_BAD_ARG;
    if ((ldw & 3) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(scales) & 15) ||
        (reinterpret_cast<uintptr_t>(salcol) & 3))
        return CRB_ERR_BAD_ARG;
    const int row_groups = (R + 7) / 8;
    if (row_groups > 65535) return CRB_ERR_UNSUPPORTED;
    k_dequantize<<<dim3(C / kBlock, row_groups), 256, 0, st>>>(W, R, C, ldw, technique, b1, lm, salcol, b2, b2_off,
                                                              b2_pitch, scales);
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
