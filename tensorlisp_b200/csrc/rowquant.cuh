// The Q8_K block quantizer shared by the row-producing kernels (k_fused.cu) and the attention epilogue (k_attn.cu).
#pragma once
#include <cuda_fp16.h>

#include "kernels.h"

namespace tlb {

__device__ __forceinline__ int nearest_int_f(float v) {
    float t = __fadd_rn(v, 12582912.f);
    return (__float_as_int(t) & 0x007fffff) - 0x00400000;
}


// Q8_K quantization of one 256-value block held by a warp (lane l: values l*8 .. l*8+7), its optional f32
// copy, and its slice of the tensor-core operand blob (quantize_row_q8_K_ref, ggml-quants.c:2768-2805)
__device__ __forceinline__ void rq_quant_block(const RowQuantArgs &p, int n, int sb, int nblk, int lane, float (&v)[8]) {
    char *ob = (char *)p.out;
    const int64_t K = p.K;
    const int64_t k0 = (int64_t)sb * 256 + lane * 8;
    int8_t *qs = (int8_t *)(ob + p.qs_off);
    float *ds = (float *)(ob + p.d_off);
    int16_t *bsums = (int16_t *)(ob + p.bsum_off);
    if (p.y_out) {
        *reinterpret_cast<float4 *>(p.y_out + n * p.ld_y + k0) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p.y_out + n * p.ld_y + k0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    float amax = 0.f, mx = 0.f;
    int idx = 512;
#pragma unroll
    for (int e = 0; e < 8; e++)
        if (fabsf(v[e]) > amax) { amax = fabsf(v[e]); mx = v[e]; idx = lane * 8 + e; }
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, s), om = __shfl_xor_sync(0xffffffffu, mx, s);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, s);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
    }
    int q[8];
    float d = 0.f;
    if (amax == 0.f) {
#pragma unroll
        for (int e = 0; e < 8; e++) q[e] = 0;
    } else {
        const float iscale = __fdiv_rn(-127.f, mx);
#pragma unroll
        for (int e = 0; e < 8; e++) q[e] = min(127, nearest_int_f(__fmul_rn(iscale, v[e])));
        d = __fdiv_rn(1.f, iscale);
    }
    int s8 = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) s8 += q[e];
    const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
    uint2 packed;
    packed.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    packed.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(qs + (size_t)n * K + k0) = packed;
    if ((lane & 1) == 0) bsums[(size_t)n * (K / 16) + sb * 16 + (lane >> 1)] = (int16_t)s16;
    if (lane == 0) ds[(size_t)n * (K / 256) + sb] = d;
    if (p.npad == MM_FOLD_NPAD) {
        // operand of the folded-scale prompt GEMM: f16(code x scale), blobs of 256 columns x 64 elements of K, natural order
        const int64_t kk = (int64_t)sb * 256 + lane * 8;
        uint8_t *o = (uint8_t *)ob + p.blob_off + ((size_t)(n >> 8) * (size_t)(K / 64) + (size_t)(kk >> 6)) * 32768 + (size_t)((n & 255) >> 3) * 1024 +
                     (size_t)((kk & 63) >> 3) * 128 + (size_t)(n & 7) * 16;
        uint32_t h[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const __half2 t = __floats2half2_rn(__fmul_rn((float)q[2 * e], d), __fmul_rn((float)q[2 * e + 1], d));
            h[e] = *reinterpret_cast<const uint32_t *>(&t);
        }
        *reinterpret_cast<uint4 *>(o) = make_uint4(h[0], h[1], h[2], h[3]);
    } else if (p.npad > 0) {
        // tensor-core operand: this lane's 8 codes are K chunk `lane` of column n, in the order
        // (0, 2, 1, 3, 4, 6, 5, 7) in which the weight nibbles come out of a 32-bit word
        const int ch = n / p.npad, nl = n % p.npad;   // blobs: [chunk of npad columns][block]
        uint8_t *o = (uint8_t *)ob + p.blob_off + ((size_t)ch * nblk + sb) * p.blob_bytes;
        __half2 h[4];
        h[0] = __floats2half2_rn((float)q[0], (float)q[2]);
        h[1] = __floats2half2_rn((float)q[1], (float)q[3]);
        h[2] = __floats2half2_rn((float)q[4], (float)q[6]);
        h[3] = __floats2half2_rn((float)q[5], (float)q[7]);
        *reinterpret_cast<uint4 *>(o + (size_t)(nl / 8) * 4096 + lane * 128 + (nl % 8) * 16) = *reinterpret_cast<const uint4 *>(h);
        if ((lane & 1) == 0)
            *reinterpret_cast<__half *>(o + (size_t)p.npad * 512 + (size_t)(nl / 8) * 256 + (lane >> 4) * 128 + (nl % 8) * 16 + ((lane >> 1) & 7) * 2) = __float2half_rn((float)s16);
        if (lane == 0) reinterpret_cast<float *>(o + (size_t)p.npad * 544)[nl] = d;
    }
}

}  // namespace tlb
