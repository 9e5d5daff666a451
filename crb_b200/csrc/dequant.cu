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
    // one warp per (row, block): lane l rebuilds columns 4 l .. 4 l + 3 of the block
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = C / kBlock;
    const long long unit = (long long)blockIdx.x * 8 + warp;
    if (unit >= (long long)R * nblk) return;
    const int row = (int)(unit / nblk), blk = (int)(unit % nblk);
    const int col = blk * kBlock + 4 * lane;
    const float* sc = scales + ((size_t)blk * R + row) * 8;
    float s[8];
    {
        const float4 s0 = *reinterpret_cast<const float4*>(sc), s1 = *reinterpret_cast<const float4*>(sc + 4);
        s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
    }
    const size_t bit_base = (size_t)row * (C / 8) + (col >> 3);
    const unsigned sh = (lane & 1) * 4;                       // this lane's four bits inside the byte
    const unsigned v1 = (b1[bit_base] >> sh) & 15u, vg = (lm[bit_base] >> sh) & 15u;
    const uchar4 scol = *reinterpret_cast<const uchar4*>(salcol + col);
    const unsigned char sk[4] = {scol.x, scol.y, scol.z, scol.w};
    const unsigned char* b2row = b2 + b2_off[blk] + (size_t)row * b2_pitch[blk];
    float q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float B1 = ((v1 >> e) & 1u) ? 1.f : -1.f;
        if (sk[e] == 255) {
            const int g = (vg >> e) & 1u;                     // 0 low, 1 mid
            q[e] = __fadd_rn(s[2 * g + 1] * B1, s[2 * g]);
        } else {
            const float B2 = ((b2row[sk[e] >> 3] >> (sk[e] & 7)) & 1u) ? 1.f : -1.f;
            if (technique == CRB_TECH_BRAQ) {
                const float y1 = __fadd_rn(s[5] * B1, s[4]);
                q[e] = __fadd_rn(y1, __fadd_rn(s[7] * B2, s[6]));
            } else {
                q[e] = __fadd_rn(__fadd_rn(s[4], __fmul_rn(s[5], B1)), __fmul_rn(s[6], B2));
            }
        }
    }
    *reinterpret_cast<float4*>(W + (int64_t)row * ldw + col) = make_float4(q[0], q[1], q[2], q[3]);
}

int dequantize_launch(float* W, int R, int C, int64_t ldw, int technique, const unsigned char* b1,
                      const unsigned char* lm, const unsigned char* salcol, const unsigned char* b2,
                      const long long* b2_off, const int* b2_pitch, const float* scales, cudaStream_t st) {
    if (!W || !b1 || !lm || !salcol || !b2 || !b2_off || !b2_pitch || !scales || R <= 0 || C <= 0) return CRB_ERR_BAD_ARG;
    if (C % kBlock) return CRB_ERR_UNSUPPORTED;
    if (technique < CRB_TECH_BRAQ || technique > CRB_TECH_CRB) return CRB_ERR_BAD_ARG;
    if ((ldw & 3) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(scales) & 15) ||
        (reinterpret_cast<uintptr_t>(salcol) & 3))
        return CRB_ERR_BAD_ARG;
    const long long units = (long long)R * (C / kBlock);
    const long long ctas = (units + 7) / 8;
    if (ctas > 0x7fffffffLL) return CRB_ERR_UNSUPPORTED;
    k_dequantize<<<(unsigned)ctas, 256, 0, st>>>(W, R, C, ldw, technique, b1, lm, salcol, b2, b2_off, b2_pitch, scales);
    CRB_LAUNCHED();
    return CRB_OK;
}

}  // namespace crb
