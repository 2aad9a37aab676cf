// Element decoders of ggml's block-quantized types (reference: crates/kernels/src/cuda/native/common.cuh:169-263, which
// follows vendor/ggml/src/ggml-quants.c dequantize_row_*; block layouts vendor/ggml/src/ggml-common.h). dq_elem returns
// element i0 of a row; every product and sum is rounded on its own (no fused multiply-add), in the order the
// reference's CPU code takes, so a decoded value has the bits ggml's dequantizer gives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "../../include/tlb200.h"

namespace tlb {

__device__ __forceinline__ float ld_elem(const uint8_t *p, uint32_t ty) {
    switch (ty) {
        case TLB_TYPE_F32: return *reinterpret_cast<const float *>(p);
        case TLB_TYPE_F16: return __half2float(*reinterpret_cast<const __half *>(p));
        case TLB_TYPE_BF16: return __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(p));
        case TLB_TYPE_I32: return (float)*reinterpret_cast<const int32_t *>(p);
        case TLB_TYPE_I64: return (float)*reinterpret_cast<const int64_t *>(p);
        default: return 0.f;
    }
}

__device__ __forceinline__ float dq_f16(const uint8_t *p) { return __half2float(__ushort_as_half((uint16_t)(p[0] | (p[1] << 8)))); }

// 6-bit scale and min of sub-block j of a Q4_K / Q5_K super-block (get_scale_min_k4, ggml-quants.c:880-887)
__device__ __forceinline__ void dq_scale_min_k4(int j, const uint8_t *s, int &sc, int &mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

__device__ __forceinline__ bool is_quant(uint32_t ty) {
    switch (ty) {
        case TLB_TYPE_Q4_0: case TLB_TYPE_Q4_1: case TLB_TYPE_Q5_0: case TLB_TYPE_Q5_1: case TLB_TYPE_Q8_0:
        case TLB_TYPE_Q2_K: case TLB_TYPE_Q3_K: case TLB_TYPE_Q4_K: case TLB_TYPE_Q5_K: case TLB_TYPE_Q6_K: return true;
        default: return false;
    }
}

__device__ __forceinline__ float dq_elem(const uint8_t *row, uint32_t ty, int64_t i0) {
    switch (ty) {
        case TLB_TYPE_Q8_0: {   // {f16 d; i8 qs[32]}
            const uint8_t *b = row + (i0 >> 5) * 34;
            return __fmul_rn((float)reinterpret_cast<const int8_t *>(b + 2)[i0 & 31], dq_f16(b));
        }
        case TLB_TYPE_Q4_0: {   // {f16 d; u8 qs[16]}: low nibbles are elements 0..15, high nibbles 16..31
            const uint8_t *b = row + (i0 >> 5) * 18;
            const int j = (int)(i0 & 31);
            const int q = j < 16 ? (b[2 + j] & 0x0F) : (b[2 + j - 16] >> 4);
            return __fmul_rn((float)(q - 8), dq_f16(b));
        }
        case TLB_TYPE_Q4_1: {   // {f16 d, m; u8 qs[16]}: x * d + m
            const uint8_t *b = row + (i0 >> 5) * 20;
            const int j = (int)(i0 & 31);
            const int q = j < 16 ? (b[4 + j] & 0x0F) : (b[4 + j - 16] >> 4);
            return __fadd_rn(__fmul_rn((float)q, dq_f16(b)), dq_f16(b + 2));
        }
        case TLB_TYPE_Q5_0:     // {f16 d; u8 qh[4]; u8 qs[16]}: fifth bit of element j in bit j of qh
        case TLB_TYPE_Q5_1: {   // {f16 d, m; u8 qh[4]; u8 qs[16]}
            const bool one = ty == TLB_TYPE_Q5_1;
            const uint8_t *b = row + (i0 >> 5) * (one ? 24 : 22);
            const uint8_t *hb = b + (one ? 4 : 2), *qs = hb + 4;
            const uint32_t qh = (uint32_t)hb[0] | ((uint32_t)hb[1] << 8) | ((uint32_t)hb[2] << 16) | ((uint32_t)hb[3] << 24);
            const int j = (int)(i0 & 31);
            const int q = (j < 16 ? (qs[j] & 0x0F) : (qs[j - 16] >> 4)) | (int)(((qh >> j) & 1u) << 4);
            if (one) return __fadd_rn(__fmul_rn((float)q, dq_f16(b)), dq_f16(b + 2));
            return __fmul_rn((float)(q - 16), dq_f16(b));
        }
        case TLB_TYPE_Q2_K: {   // {u8 scales[16] (4-bit scale, 4-bit min); u8 qs[64]; f16 d, dmin}
            const uint8_t *b = row + (i0 >> 8) * 84;
            const int e = (int)(i0 & 255), n = e >> 7, j = (e >> 5) & 3, sub = (e >> 4) & 1, l = e & 15;
            const uint8_t sc = b[n * 8 + 2 * j + sub];
            const int q = (b[16 + n * 32 + sub * 16 + l] >> (2 * j)) & 3;
            const float dl = __fmul_rn(dq_f16(b + 80), (float)(sc & 0xF)), ml = __fmul_rn(dq_f16(b + 82), (float)(sc >> 4));
            return __fsub_rn(__fmul_rn(dl, (float)q), ml);
        }
        case TLB_TYPE_Q3_K: {   // {u8 hmask[32]; u8 qs[64]; u8 scales[12] (6-bit, packed); f16 d}
            const uint8_t *b = row + (i0 >> 8) * 110;
            const int e = (int)(i0 & 255), n = e >> 7, j = (e >> 5) & 3, sub = (e >> 4) & 1, l = e & 15;
            const int is = n * 8 + 2 * j + sub, g = is >> 2, i = is & 3;
            const uint8_t *s = b + 96;
            const int lo = g < 2 ? (s[4 * g + i] & 0xF) : (s[4 * (g - 2) + i] >> 4);
            const int hi = (s[8 + i] >> (2 * g)) & 3;
            const int scale = (int)(int8_t)(lo | (hi << 4)) - 32;
            const int q = ((b[32 + n * 32 + sub * 16 + l] >> (2 * j)) & 3) - ((b[sub * 16 + l] & (1 << (4 * n + j))) ? 0 : 4);
            return __fmul_rn(__fmul_rn(dq_f16(b + 108), (float)scale), (float)q);
        }
        case TLB_TYPE_Q4_K: {   // {f16 d, dmin; u8 scales[12]; u8 qs[128]}
            const uint8_t *b = row + (i0 >> 8) * 144;
            const int e = (int)(i0 & 255), j = e >> 5, l = e & 31;
            int sc, mn;
            dq_scale_min_k4(j, b + 4, sc, mn);
            const int q = (b[16 + (j >> 1) * 32 + l] >> ((j & 1) * 4)) & 0xF;
            return __fsub_rn(__fmul_rn(__fmul_rn(dq_f16(b), (float)sc), (float)q), __fmul_rn(dq_f16(b + 2), (float)mn));
        }
        case TLB_TYPE_Q5_K: {   // {f16 d, dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}
            const uint8_t *b = row + (i0 >> 8) * 176;
            const int e = (int)(i0 & 255), j = e >> 5, l = e & 31;
            int sc, mn;
            dq_scale_min_k4(j, b + 4, sc, mn);
            const int q = ((b[48 + (j >> 1) * 32 + l] >> ((j & 1) * 4)) & 0xF) + ((b[16 + l] & (1 << j)) ? 16 : 0);
            return __fsub_rn(__fmul_rn(__fmul_rn(dq_f16(b), (float)sc), (float)q), __fmul_rn(dq_f16(b + 2), (float)mn));
        }
        case TLB_TYPE_Q6_K: {   // {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}
            const uint8_t *b = row + (i0 >> 8) * 210;
            const int e = (int)(i0 & 255), n = e >> 7, quarter = (e >> 5) & 3, l = e & 31;
            const uint8_t lo = b[n * 64 + (quarter & 1) * 32 + l];
            const int q = (int)(int8_t)(((quarter & 2) ? (lo >> 4) : (lo & 0xF)) | (((b[128 + n * 32 + l] >> (2 * quarter)) & 3) << 4)) - 32;
            const int sc = (int)reinterpret_cast<const int8_t *>(b + 192)[n * 8 + (l >> 4) + 2 * quarter];
            return __fmul_rn(__fmul_rn(dq_f16(b + 208), (float)sc), (float)q);
        }
        default: return ld_elem(row + i0 * (ty == TLB_TYPE_F32 || ty == TLB_TYPE_I32 ? 4 : (ty == TLB_TYPE_I64 ? 8 : 2)), ty);
    }
}

}  // namespace tlb
