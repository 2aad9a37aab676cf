// Row quantizers, bit-exact with the reference's ggml build.
//
// Weights (`tl quantize`, crates/tensorlisp/src/dtype.rs:98-124 -> ggml_quantize_chunk):
//   quantize_row_q8_0_ref  vendor/ggml/src/ggml-quants.c:276-299
//   quantize_row_q4_0_ref  vendor/ggml/src/ggml-quants.c:113-148
//   quantize_row_q4_K_ref  vendor/ggml/src/ggml-quants.c:1457-1527 (+ make_qkx2_quants :799-878)
// Activations of MUL_MAT (ggml-cpu quantizes src1 to the weight type's vec_dot_type,
// vendor/ggml/src/ggml-cpu/ggml-cpu.c:1272-1357):
//   quantize_row_q8_0 (roundf)                      ggml-quants.c:276-299
//   quantize_row_q8_K_ref (magic-number rounding)   ggml-quants.c:2768-2805
//
// The reference is built without FMA contraction, and the Q4_K scale search depends on every
// intermediate rounding, so this file is compiled with -fmad=false and spells the order of every
// float operation with round-to-nearest intrinsics. Division and sqrt are the IEEE versions.
#include <cuda_fp16.h>

#include "kernels.h"

namespace tlb {

__device__ __forceinline__ int nearest_int(float v) {  // ggml-quants.c:621-626
    float t = __fadd_rn(v, 12582912.f);
    return (__float_as_int(t) & 0x007fffff) - 0x00400000;
}

// ------------------------------------------------------------------ Q8_0 (weights and activations)
// 8 lanes per 32-element block; lane holds 4 consecutive values.
__global__ void __launch_bounds__(256) k_quantize_q8_0(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nblocks) {
    const int64_t gid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    int64_t b = gid >> 3;
    const int l = (int)(gid & 7);
    const bool live = b < nblocks;
    if (!live) b = nblocks - 1;
    const float4 v = *reinterpret_cast<const float4 *>(x + b * 32 + l * 4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d = __fdiv_rn(amax, 127.f);
    const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q0 = (int)roundf(__fmul_rn(v.x, id)), q1 = (int)roundf(__fmul_rn(v.y, id));
    const int q2 = (int)roundf(__fmul_rn(v.z, id)), q3 = (int)roundf(__fmul_rn(v.w, id));
    if (!live) return;
    uint16_t *o = reinterpret_cast<uint16_t *>(y + b * 34);  // blocks are 2-byte aligned
    if (l == 0) o[0] = __half_as_ushort(__float2half_rn(d));
    o[1 + 2 * l] = (uint16_t)((q0 & 0xff) | ((q1 & 0xff) << 8));
    o[2 + 2 * l] = (uint16_t)((q2 & 0xff) | ((q3 & 0xff) << 8));
}

// ------------------------------------------------------------------ Q4_0
// 8 lanes per block; lanes 0..3 hold elements 0..15 (low nibbles), lanes 4..7 elements 16..31.
__global__ void __launch_bounds__(256) k_quantize_q4_0(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nblocks) {
    const int64_t gid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    int64_t b = gid >> 3;
    const int l = (int)(gid & 7);
    const bool live = b < nblocks;
    if (!live) b = nblocks - 1;
    const float4 v = *reinterpret_cast<const float4 *>(x + b * 32 + l * 4);
    // first element (lowest index) with the largest magnitude: `if (amax < fabsf(v))` is strict
    float amax = 0.0f, mx = 0.0f;
    int idx = 0;
    const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++)
        if (amax < fabsf(vv[i])) { amax = fabsf(vv[i]); mx = vv[i]; idx = l * 4 + i; }
    if (amax == 0.0f) idx = 64;  // never selected against a real maximum
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, s);
        const float om = __shfl_xor_sync(0xffffffffu, mx, s);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, s);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
    }
    const float d = __fdiv_rn(mx, -8.f);
    const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.0f;
    uint32_t nib = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int q = (int)(signed char)(int)__fadd_rn(__fmul_rn(vv[i], id), 8.5f);
        q = q > 15 ? 15 : q;
        nib |= (uint32_t)(q & 0xff) << (8 * i);
    }
    const uint32_t hi = __shfl_down_sync(0xffffffffu, nib, 4, 8);
    if (!live || l >= 4) return;
    const uint32_t bytes = nib | (hi << 4);
    uint16_t *o = reinterpret_cast<uint16_t *>(y + b * 18);
    if (l == 0) o[0] = __half_as_ushort(__float2half_rn(d));
    o[1 + 2 * l] = (uint16_t)(bytes & 0xffff);
    o[2 + 2 * l] = (uint16_t)(bytes >> 16);
}

// ------------------------------------------------------------------ Q4_K
// One thread per 32-element sub-block (the scale search is a chain of ordered f32 reductions in
// which every candidate depends on the previous winner, so it cannot be split further), eight
// threads per 256-element super-block, 32 super-blocks per CTA.
__global__ void __launch_bounds__(256) k_quantize_q4_K(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nsuper) {
    __shared__ uint8_t Ls[32][256];
    const int tid = threadIdx.x;
    const int sub = tid & 7;
    const int sl = tid >> 3;
    int64_t sb = (int64_t)blockIdx.x * 32 + sl;
    const bool live = sb < nsuper;
    if (!live) sb = nsuper - 1;
    const float *xs = x + sb * 256 + sub * 32;
    float v[32];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 t = reinterpret_cast<const float4 *>(xs)[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    float sum_x2 = 0.f;
#pragma unroll
    for (int l = 0; l < 32; l++) sum_x2 = __fadd_rn(sum_x2, __fmul_rn(v[l], v[l]));
    const float av_x = __fsqrt_rn(__fdiv_rn(sum_x2, 32.f));
#define W(i) __fadd_rn(av_x, fabsf(v[i]))

    // make_qkx2_quants(32, 15, x, weights, L, &the_min, Laux, -1, 0.1, 20, false)
    float mn = v[0], mx = v[0];
    float sum_w = W(0);
    float sum_x = __fmul_rn(sum_w, v[0]);
#pragma unroll
    for (int i = 1; i < 32; i++) {
        if (v[i] < mn) mn = v[i];
        if (v[i] > mx) mx = v[i];
        const float w = W(i);
        sum_w = __fadd_rn(sum_w, w);
        sum_x = __fadd_rn(sum_x, __fmul_rn(w, v[i]));
    }
    if (mn > 0.f) mn = 0.f;
    float scale = 0.f;
    // (iscale, min) that produced the winning codes, to recompute them if they are needed
    float L_iscale = 0.f, L_min = 0.f;
    bool flat = (mx == mn);
    if (!flat) {
        float iscale = __fdiv_rn(15.f, __fsub_rn(mx, mn));
        scale = __fdiv_rn(1.f, iscale);
        float best = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            int l = nearest_int(__fmul_rn(iscale, __fsub_rn(v[i], mn)));
            l = max(0, min(15, l));
            float diff = __fsub_rn(__fadd_rn(__fmul_rn(scale, (float)l), mn), v[i]);
            diff = __fmul_rn(diff, diff);
            best = __fadd_rn(best, __fmul_rn(W(i), diff));
        }
        L_iscale = iscale;
        L_min = mn;
        for (int is = 0; is <= 20; is++) {
            iscale = __fdiv_rn(__fadd_rn(__fadd_rn(-1.f, __fmul_rn(0.1f, (float)is)), 15.f), __fsub_rn(mx, mn));
            float sum_l = 0.f, sum_l2 = 0.f, sum_xl = 0.f;
            uint32_t codes[4] = {0, 0, 0, 0};  // 32 nibbles of this candidate
#pragma unroll
            for (int i = 0; i < 32; i++) {
                int l = nearest_int(__fmul_rn(iscale, __fsub_rn(v[i], mn)));
                l = max(0, min(15, l));
                codes[i >> 3] |= (uint32_t)l << (4 * (i & 7));
                const float wl = __fmul_rn(W(i), (float)l);
                sum_l = __fadd_rn(sum_l, wl);
                sum_l2 = __fadd_rn(sum_l2, __fmul_rn(wl, (float)l));
                sum_xl = __fadd_rn(sum_xl, __fmul_rn(wl, v[i]));
            }
            const float D = __fsub_rn(__fmul_rn(sum_w, sum_l2), __fmul_rn(sum_l, sum_l));
            if (D > 0.f) {
                float this_scale = __fdiv_rn(__fsub_rn(__fmul_rn(sum_w, sum_xl), __fmul_rn(sum_x, sum_l)), D);
                float this_min = __fdiv_rn(__fsub_rn(__fmul_rn(sum_l2, sum_x), __fmul_rn(sum_l, sum_xl)), D);
                if (this_min > 0.f) {
                    this_min = 0.f;
                    this_scale = __fdiv_rn(sum_xl, sum_l2);
                }
                float err = 0.f;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float l = (float)((codes[i >> 3] >> (4 * (i & 7))) & 15u);
                    float diff = __fsub_rn(__fadd_rn(__fmul_rn(this_scale, l), this_min), v[i]);
                    diff = __fmul_rn(diff, diff);
                    err = __fadd_rn(err, __fmul_rn(W(i), diff));
                }
                if (err < best) {
                    L_iscale = iscale;
                    L_min = mn;
                    best = err;
                    scale = this_scale;
                    mn = this_min;
                }
            }
        }
    }
    const float the_min = -mn;

    // super-block maxima over the 8 sub-block threads (the reference starts both at 0)
    float max_scale = fmaxf(scale, 0.f), max_min = fmaxf(the_min, 0.f);
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
        max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, s));
        max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, s));
    }
    const float inv_scale = max_scale > 0.f ? __fdiv_rn(63.f, max_scale) : 0.f;
    const float inv_min = max_min > 0.f ? __fdiv_rn(63.f, max_min) : 0.f;
    uint32_t ls = (uint32_t)nearest_int(__fmul_rn(inv_scale, scale)) & 0xffu;
    uint32_t lm = (uint32_t)nearest_int(__fmul_rn(inv_min, the_min)) & 0xffu;
    ls = min(63u, ls);
    lm = min(63u, lm);
    const __half dh = __float2half_rn(__fdiv_rn(max_scale, 63.f));
    const __half dmh = __float2half_rn(__fdiv_rn(max_min, 63.f));

    // final codes against the stored (rounded) scales
    const float d = __fmul_rn(__half2float(dh), (float)ls);
    uint8_t *Lrow = &Ls[sl][sub * 32];
    if (d != 0.f) {
        const float dm = __fmul_rn(__half2float(dmh), (float)lm);
#pragma unroll
        for (int i = 0; i < 32; i++) {
            int l = nearest_int(__fdiv_rn(__fadd_rn(v[i], dm), d));
            Lrow[i] = (uint8_t)max(0, min(15, l));
        }
    } else {
        // the reference keeps the search's codes in this case
#pragma unroll
        for (int i = 0; i < 32; i++) {
            int l = 0;
            if (!flat) {
                l = nearest_int(__fmul_rn(L_iscale, __fsub_rn(v[i], L_min)));
                l = max(0, min(15, l));
            }
            Lrow[i] = (uint8_t)l;
        }
    }
    // gather the eight (ls, lm) pairs of the super-block
    uint32_t lsv[8], lmv[8];
    const int base = (tid & 31) & ~7;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        lsv[j] = __shfl_sync(0xffffffffu, ls, base + j);
        lmv[j] = __shfl_sync(0xffffffffu, lm, base + j);
    }
    __syncwarp();
    if (!live) return;
    uint8_t *out = y + sb * 144;
    if (sub == 0) {
        uint32_t sc[3] = {0, 0, 0};
        uint8_t *scb = reinterpret_cast<uint8_t *>(sc);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (j < 4) {
                scb[j] |= (uint8_t)lsv[j];
                scb[j + 4] |= (uint8_t)lmv[j];
            } else {
                scb[j + 4] = (uint8_t)((lsv[j] & 0xF) | ((lmv[j] & 0xF) << 4));
                scb[j - 4] |= (uint8_t)((lsv[j] >> 4) << 6);
                scb[j] |= (uint8_t)((lmv[j] >> 4) << 6);
            }
        }
        uint4 hdr;
        hdr.x = (uint32_t)__half_as_ushort(dh) | ((uint32_t)__half_as_ushort(dmh) << 16);
        hdr.y = sc[0]; hdr.z = sc[1]; hdr.w = sc[2];
        *reinterpret_cast<uint4 *>(out) = hdr;
    }
    // qs bytes [16*sub, 16*sub+16): chunk c = sub/2 pairs sub-blocks 2c (low) and 2c+1 (high)
    const int c = sub >> 1, l0 = (sub & 1) * 16;
    const uint8_t *lo = &Ls[sl][64 * c + l0], *hi = &Ls[sl][64 * c + 32 + l0];
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t a = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) a |= (uint32_t)(lo[4 * k + e] | (hi[4 * k + e] << 4)) << (8 * e);
        w[k] = a;
    }
    *reinterpret_cast<uint4 *>(out + 16 + 16 * sub) = make_uint4(w[0], w[1], w[2], w[3]);
#undef W
}

// ------------------------------------------------------------------ F16 rows
__global__ void k_f32_to_f16(const float *__restrict__ x, __half *__restrict__ y, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(x[i]);
}

// ------------------------------------------------------------------ activations for MUL_MAT
// Internal layout of a quantized activation matrix [K, N] (see ActLayout in kernels.h):
//   qs int8 [N][K] | d f32 [N][K/blk] | (Q8_K only) bsums int16 [N][K/16]
// Q8_0 flavour: d is the f16-rounded scale widened back to f32 (what the dot product reads).
// x may be strided: column n starts at x + n*ldx (elements).
__global__ void __launch_bounds__(256) k_act_q8_0(const float *__restrict__ x, int64_t ldx, int8_t *__restrict__ qs,
                                                   float *__restrict__ ds, int64_t K, int64_t N) {
    const int64_t gid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t nblk = K / 32 * N;
    int64_t b = gid >> 3;
    const int l = (int)(gid & 7);
    const bool live = b < nblk;
    if (!live) b = nblk - 1;
    const int64_t n = b / (K / 32), kb = b % (K / 32);
    const float4 v = *reinterpret_cast<const float4 *>(x + n * ldx + kb * 32 + l * 4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d = __fdiv_rn(amax, 127.f);
    const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q0 = (int)roundf(__fmul_rn(v.x, id)), q1 = (int)roundf(__fmul_rn(v.y, id));
    const int q2 = (int)roundf(__fmul_rn(v.z, id)), q3 = (int)roundf(__fmul_rn(v.w, id));
    if (!live) return;
    *reinterpret_cast<uint32_t *>(qs + n * K + kb * 32 + l * 4) =
        (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
    if (l == 0) ds[n * (K / 32) + kb] = __half2float(__float2half_rn(d));
}

// One warp per 256-element block; lane holds 8 consecutive values (half of a 16-element bsum group).
__global__ void __launch_bounds__(256) k_act_q8_K(const float *__restrict__ x, int64_t ldx, int8_t *__restrict__ qs,
                                                   float *__restrict__ ds, int16_t *__restrict__ bsums, int64_t K,
                                                   int64_t N) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = K / 256 * N;
    int64_t b = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const bool live = b < nblk;
    if (!live) b = nblk - 1;
    const int64_t n = b / (K / 256), kb = b % (K / 256);
    const float *xs = x + n * ldx + kb * 256 + lane * 8;
    const float4 a = reinterpret_cast<const float4 *>(xs)[0], c = reinterpret_cast<const float4 *>(xs)[1];
    const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    // first element with the largest magnitude (`if (ax > amax)` is strict)
    float amax = 0.f, mx = 0.f;
    int idx = 512;
#pragma unroll
    for (int i = 0; i < 8; i++)
        if (fabsf(v[i]) > amax) { amax = fabsf(v[i]); mx = v[i]; idx = lane * 8 + i; }
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, s);
        const float om = __shfl_xor_sync(0xffffffffu, mx, s);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, s);
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
    }
    int q[8];
    float d = 0.f;
    if (amax == 0.f) {
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = 0;
    } else {
        const float iscale = __fdiv_rn(-127.f, mx);
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = min(127, nearest_int(__fmul_rn(iscale, v[i])));
        d = __fdiv_rn(1.f, iscale);
    }
    int s8 = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) s8 += q[i];
    const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
    if (!live) return;
    uint2 packed;
    packed.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    packed.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(qs + n * K + kb * 256 + lane * 8) = packed;
    if ((lane & 1) == 0) bsums[n * (K / 16) + kb * 16 + (lane >> 1)] = (int16_t)s16;
    if (lane == 0) ds[n * (K / 256) + kb] = d;
}

// ------------------------------------------------------------------ launchers
cudaError_t launch_quantize_rows(uint32_t type, const float *x, int64_t rows, int64_t n_per_row, void *y,
                                 cudaStream_t st) {
    const int64_t n = rows * n_per_row;
    if (n == 0) return cudaSuccess;
    switch (type) {
        case TLB_TYPE_Q8_0: {
            const int64_t nb = n / 32;
            k_quantize_q8_0<<<(unsigned)((nb * 8 + 255) / 256), 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_Q4_0: {
            const int64_t nb = n / 32;
            k_quantize_q4_0<<<(unsigned)((nb * 8 + 255) / 256), 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_Q4_K: {
            const int64_t nb = n / 256;
            k_quantize_q4_K<<<(unsigned)((nb + 31) / 32), 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_F16:
            k_f32_to_f16<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, (__half *)y, n);
            break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

ActLayout act_layout(int kind, int64_t K, int64_t N) {
    ActLayout a;
    a.kind = kind;
    a.K = K;
    a.N = N;
    a.qs_off = 0;
    a.d_off = (uint64_t)((K * N + 255) / 256 * 256);
    const int64_t blk = kind == ACT_Q8_K ? 256 : 32;
    const uint64_t dbytes = (uint64_t)(K / blk * N * 4);
    a.bsum_off = a.d_off + (dbytes + 255) / 256 * 256;
    a.bytes = a.bsum_off + (kind == ACT_Q8_K ? (uint64_t)((K / 16 * N * 2 + 255) / 256 * 256) : 0);
    return a;
}

cudaError_t launch_act_quantize(const ActLayout &a, const float *x, int64_t ldx, void *out, cudaStream_t st) {
    if (a.K == 0 || a.N == 0) return cudaSuccess;
    char *o = (char *)out;
    if (a.kind == ACT_Q8_0) {
        const int64_t nb = a.K / 32 * a.N;
        k_act_q8_0<<<(unsigned)((nb * 8 + 255) / 256), 256, 0, st>>>(x, ldx, (int8_t *)(o + a.qs_off), (float *)(o + a.d_off), a.K, a.N);
    } else {
        const int64_t nb = a.K / 256 * a.N;
        k_act_q8_K<<<(unsigned)((nb + 7) / 8), 256, 0, st>>>(x, ldx, (int8_t *)(o + a.qs_off), (float *)(o + a.d_off),
                                                            (int16_t *)(o + a.bsum_off), a.K, a.N);
    }
    return cudaGetLastError();
}

}  // namespace tlb
