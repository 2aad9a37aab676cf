// Row quantizers, bit-exact with the reference's ggml build.
//
// Weights (`tl quantize`, crates/tensorlisp/src/dtype.rs:98-124 -> ggml_quantize_chunk):
//   quantize_row_q8_0_ref  vendor/ggml/src/ggml-quants.c:276-299
//   quantize_row_q4_0_ref  vendor/ggml/src/ggml-quants.c:113-148
//   quantize_row_q4_K_ref  vendor/ggml/src/ggml-quants.c:1457-1527 (+ make_qkx2_quants :799-878)
//   quantize_row_q4_1_ref / q5_0_ref / q5_1_ref       ggml-quants.c:150-273
//   quantize_row_q2_K_ref  ggml-quants.c:891-958      (make_qkx2_quants on 16 elements, absolute error)
//   quantize_row_q3_K_ref  ggml-quants.c:1229-1303    (+ make_q3_quants :697-754)
//   quantize_row_q5_K_ref  ggml-quants.c:1644-1727    (make_qkx2_quants with 5-bit codes)
//   quantize_row_q6_K_ref  ggml-quants.c:1869-1937    (+ make_qx_quants :628-695)
//   f32 -> bf16            ggml-impl.h ggml_compute_fp32_to_bf16
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

// ------------------------------------------------------------------ the (scale, min) search of the K-quants
// make_qkx2_quants for one group of N values held in registers: codes 0..NMAX, weights av_x + |x| (av_x = 0 gives the
// plain |x| of Q2_K), squared or absolute (MAD) error. The search is a chain of ordered f32 reductions in which every
// candidate depends on the previous winner, so one thread runs it. Instead of the winning codes the (iscale, min) that
// produced them are returned: the caller recomputes the codes in the rare case it needs them.
struct ScaleMin {
    float scale, the_min, L_iscale, L_min;
    bool flat;
};

template <int N, int NMAX, bool MAD>
__device__ __forceinline__ ScaleMin search_scale_min(const float (&v)[N], float av_x, float rmin, int nstep) {
#define W(i) __fadd_rn(av_x, fabsf(v[i]))
    float mn = v[0], mx = v[0];
    float sum_w = W(0);
    float sum_x = __fmul_rn(sum_w, v[0]);
#pragma unroll
    for (int i = 1; i < N; i++) {
        if (v[i] < mn) mn = v[i];
        if (v[i] > mx) mx = v[i];
        const float w = W(i);
        sum_w = __fadd_rn(sum_w, w);
        sum_x = __fadd_rn(sum_x, __fmul_rn(w, v[i]));
    }
    if (mn > 0.f) mn = 0.f;
    ScaleMin r;
    r.scale = 0.f;
    r.L_iscale = 0.f;
    r.L_min = 0.f;
    r.flat = (mx == mn);
    if (!r.flat) {
        float iscale = __fdiv_rn((float)NMAX, __fsub_rn(mx, mn));
        r.scale = __fdiv_rn(1.f, iscale);
        float best = 0.f;
#pragma unroll
        for (int i = 0; i < N; i++) {
            int l = nearest_int(__fmul_rn(iscale, __fsub_rn(v[i], mn)));
            l = max(0, min(NMAX, l));
            float diff = __fsub_rn(__fadd_rn(__fmul_rn(r.scale, (float)l), mn), v[i]);
            diff = MAD ? fabsf(diff) : __fmul_rn(diff, diff);
            best = __fadd_rn(best, __fmul_rn(W(i), diff));
        }
        r.L_iscale = iscale;
        r.L_min = mn;
        for (int is = 0; is <= nstep; is++) {
            iscale = __fdiv_rn(__fadd_rn(__fadd_rn(rmin, __fmul_rn(0.1f, (float)is)), (float)NMAX), __fsub_rn(mx, mn));
            float sum_l = 0.f, sum_l2 = 0.f, sum_xl = 0.f;
            uint32_t codes[N / 4];  // this candidate's codes, one byte each
#pragma unroll
            for (int i = 0; i < N / 4; i++) codes[i] = 0;
#pragma unroll
            for (int i = 0; i < N; i++) {
                int l = nearest_int(__fmul_rn(iscale, __fsub_rn(v[i], mn)));
                l = max(0, min(NMAX, l));
                codes[i >> 2] |= (uint32_t)l << (8 * (i & 3));
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
                for (int i = 0; i < N; i++) {
                    const float l = (float)((codes[i >> 2] >> (8 * (i & 3))) & 255u);
                    float diff = __fsub_rn(__fadd_rn(__fmul_rn(this_scale, l), this_min), v[i]);
                    diff = MAD ? fabsf(diff) : __fmul_rn(diff, diff);
                    err = __fadd_rn(err, __fmul_rn(W(i), diff));
                }
                if (err < best) {
                    r.L_iscale = iscale;
                    r.L_min = mn;
                    best = err;
                    r.scale = this_scale;
                    mn = this_min;
                }
            }
        }
    }
    r.the_min = -mn;
    return r;
#undef W
}

// ------------------------------------------------------------------ Q4_K and Q5_K
// One thread per 32-element sub-block, eight threads per 256-element super-block, 32 super-blocks per CTA.
// Q4_K: search with 4-bit codes, rmin -1, 20 steps; block {f16 d, dmin; u8 scales[12]; u8 qs[128]} = 144 B.
// Q5_K: 5-bit codes, rmin -0.5, 15 steps; block {f16 d, dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} = 176 B.
template <bool Q5>
__global__ void __launch_bounds__(256) k_quantize_q45_K(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                         int64_t nsuper) {
    constexpr int NMAX = Q5 ? 31 : 15;
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
    const ScaleMin r = search_scale_min<32, NMAX, false>(v, av_x, Q5 ? -0.5f : -1.f, Q5 ? 15 : 20);
    const float scale = r.scale, the_min = r.the_min;

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
            Lrow[i] = (uint8_t)max(0, min(NMAX, l));
        }
    } else {
        // the reference keeps the search's codes in this case
#pragma unroll
        for (int i = 0; i < 32; i++) {
            int l = 0;
            if (!r.flat) {
                l = nearest_int(__fmul_rn(r.L_iscale, __fsub_rn(v[i], r.L_min)));
                l = max(0, min(NMAX, l));
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
    uint8_t *out = y + sb * (Q5 ? 176 : 144);
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
    if (Q5) {
        // qh[j], j in [4*sub, 4*sub+4): bit 2c is the fifth bit of element 64c + j, bit 2c+1 that of element 64c + 32 + j
        uint32_t h = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int j = 4 * sub + e;
            uint32_t bits = 0;
#pragma unroll
            for (int c = 0; c < 4; c++)
                bits |= (uint32_t)(Ls[sl][64 * c + j] >> 4) << (2 * c) | (uint32_t)(Ls[sl][64 * c + 32 + j] >> 4) << (2 * c + 1);
            h |= bits << (8 * e);
        }
        *reinterpret_cast<uint32_t *>(out + 16 + 4 * sub) = h;
    }
    // qs bytes [16*sub, 16*sub+16): chunk c = sub/2 pairs sub-blocks 2c (low) and 2c+1 (high)
    const int c = sub >> 1, l0 = (sub & 1) * 16;
    const uint8_t *lo = &Ls[sl][64 * c + l0], *hi = &Ls[sl][64 * c + 32 + l0];
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t a = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) a |= (uint32_t)((lo[4 * k + e] & 15) | ((hi[4 * k + e] & 15) << 4)) << (8 * e);
        w[k] = a;
    }
    *reinterpret_cast<uint4 *>(out + (Q5 ? 48 : 16) + 16 * sub) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ------------------------------------------------------------------ Q4_1, Q5_0, Q5_1
// 8 lanes per 32-element block, 4 consecutive values per lane; lanes 0..3 hold elements 0..15 (low nibbles of qs),
// lanes 4..7 elements 16..31 (high nibbles). KIND 0 = Q4_1 {f16 d, m; qs[16]} 20 B, 1 = Q5_0 {f16 d; qh[4]; qs[16]}
// 22 B, 2 = Q5_1 {f16 d, m; qh[4]; qs[16]} 24 B. Bit e of qh is the fifth bit of element e.
template <int KIND>
__global__ void __launch_bounds__(256) k_quantize_q451(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nblocks) {
    const int64_t gid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    int64_t b = gid >> 3;
    const int l = (int)(gid & 7);
    const bool live = b < nblocks;
    if (!live) b = nblocks - 1;
    const float4 v = *reinterpret_cast<const float4 *>(x + b * 32 + l * 4);
    const float vv[4] = {v.x, v.y, v.z, v.w};
    float d, off = 0.f;      // code = (x - off) / d
    __half mh = __float2half_rn(0.f);
    if (KIND == 1) {
        // the signed value of the first element with the largest magnitude
        float amax = 0.0f, mx = 0.0f;
        int idx = 0;
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (amax < fabsf(vv[i])) { amax = fabsf(vv[i]); mx = vv[i]; idx = l * 4 + i; }
        if (amax == 0.0f) idx = 64;
#pragma unroll
        for (int s = 1; s < 8; s <<= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, amax, s);
            const float om = __shfl_xor_sync(0xffffffffu, mx, s);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, s);
            if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
        }
        d = __fdiv_rn(mx, -16.f);
    } else {
        // first minimum and first maximum in element order (`if (v < min)` / `if (v > max)` are strict: among equal
        // values, +0 and -0 included, the lowest index stays)
        float mn = vv[0], mx = vv[0];
        int imn = l * 4, imx = l * 4;
#pragma unroll
        for (int i = 1; i < 4; i++) {
            if (vv[i] < mn) { mn = vv[i]; imn = l * 4 + i; }
            if (vv[i] > mx) { mx = vv[i]; imx = l * 4 + i; }
        }
#pragma unroll
        for (int s = 1; s < 8; s <<= 1) {
            const float on = __shfl_xor_sync(0xffffffffu, mn, s), ox = __shfl_xor_sync(0xffffffffu, mx, s);
            const int oin = __shfl_xor_sync(0xffffffffu, imn, s), oix = __shfl_xor_sync(0xffffffffu, imx, s);
            if (on < mn || (on == mn && oin < imn)) { mn = on; imn = oin; }
            if (ox > mx || (ox == mx && oix < imx)) { mx = ox; imx = oix; }
        }
        d = __fdiv_rn(__fsub_rn(mx, mn), KIND == 0 ? 15.f : 31.f);
        off = mn;
        mh = __float2half_rn(mn);
    }
    const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.0f;
    uint32_t nib = 0, fifth = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int q;
        if (KIND == 0) q = min(15, (int)(signed char)(int)__fadd_rn(__fmul_rn(__fsub_rn(vv[i], off), id), 0.5f));
        else if (KIND == 1) q = min(31, (int)(signed char)(int)__fadd_rn(__fmul_rn(vv[i], id), 16.5f));
        else q = (int)(unsigned char)(int)__fadd_rn(__fmul_rn(__fsub_rn(vv[i], off), id), 0.5f);
        nib |= (uint32_t)(q & 0x0f) << (8 * i);
        fifth |= (uint32_t)((q >> 4) & 1) << (l * 4 + i);
    }
    if (KIND != 0) {
#pragma unroll
        for (int s = 1; s < 8; s <<= 1) fifth |= __shfl_xor_sync(0xffffffffu, fifth, s);
    }
    const uint32_t hi = __shfl_down_sync(0xffffffffu, nib, 4, 8);
    if (!live || l >= 4) return;
    const uint32_t bytes = nib | (hi << 4);
    constexpr int BLOCK = KIND == 0 ? 20 : (KIND == 1 ? 22 : 24), QS = KIND == 0 ? 2 : (KIND == 1 ? 3 : 4);  // in u16
    uint16_t *o = reinterpret_cast<uint16_t *>(y + b * BLOCK);
    if (l == 0) {
        o[0] = __half_as_ushort(__float2half_rn(d));
        if (KIND != 1) o[1] = __half_as_ushort(mh);
        if (KIND != 0) {
            o[QS - 2] = (uint16_t)(fifth & 0xffff);
            o[QS - 1] = (uint16_t)(fifth >> 16);
        }
    }
    o[QS + 2 * l] = (uint16_t)(bytes & 0xffff);
    o[QS + 2 * l + 1] = (uint16_t)(bytes >> 16);
}

// First lane of a 16-lane group (in index order) whose |s| is the largest: what a `if (fabsf(s) > amax)` scan keeps.
__device__ __forceinline__ float first_largest_magnitude16(float s, int g) {
    float a = fabsf(s);
    int idx = a > 0.f ? g : 64;   // a scan that starts at 0 never picks a zero
#pragma unroll
    for (int sh = 1; sh < 16; sh <<= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, sh);
        const float os = __shfl_xor_sync(0xffffffffu, s, sh);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, sh);
        if (oa > a || (oa == a && oi < idx)) { a = oa; s = os; idx = oi; }
    }
    return a > 0.f ? s : 0.f;
}

// ------------------------------------------------------------------ Q2_K
// One thread per 16-element group, 16 threads per super-block, 16 super-blocks per CTA.
// Block {u8 scales[16] (scale | min << 4); u8 qs[64]; f16 d, dmin} = 84 B.
__global__ void __launch_bounds__(256) k_quantize_q2_K(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nsuper) {
    __shared__ uint8_t Ls[16][256];
    const int tid = threadIdx.x, g = tid & 15, sl = tid >> 4;
    int64_t sb = (int64_t)blockIdx.x * 16 + sl;
    const bool live = sb < nsuper;
    if (!live) sb = nsuper - 1;
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 t = reinterpret_cast<const float4 *>(x + sb * 256 + g * 16)[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    const ScaleMin r = search_scale_min<16, 3, true>(v, 0.f, -0.5f, 15);
    float max_scale = fmaxf(r.scale, 0.f), max_min = fmaxf(r.the_min, 0.f);
#pragma unroll
    for (int s = 1; s < 16; s <<= 1) {
        max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, s));
        max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, s));
    }
    uint8_t scb = 0;
    __half dh = __float2half_rn(0.f), dmh = __float2half_rn(0.f);
    if (max_scale > 0.f) {
        scb = (uint8_t)nearest_int(__fmul_rn(__fdiv_rn(15.f, max_scale), r.scale));
        dh = __float2half_rn(__fdiv_rn(max_scale, 15.f));
    }
    if (max_min > 0.f) {
        scb |= (uint8_t)(nearest_int(__fmul_rn(__fdiv_rn(15.f, max_min), r.the_min)) << 4);
        dmh = __float2half_rn(__fdiv_rn(max_min, 15.f));
    }
    const float d = __fmul_rn(__half2float(dh), (float)(scb & 0xF));
    uint8_t *Lrow = &Ls[sl][g * 16];
    if (d != 0.f) {
        const float dm = __fmul_rn(__half2float(dmh), (float)(scb >> 4));
#pragma unroll
        for (int i = 0; i < 16; i++) Lrow[i] = (uint8_t)max(0, min(3, nearest_int(__fdiv_rn(__fadd_rn(v[i], dm), d))));
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++)
            Lrow[i] = r.flat ? 0 : (uint8_t)max(0, min(3, nearest_int(__fmul_rn(r.L_iscale, __fsub_rn(v[i], r.L_min)))));
    }
    __syncwarp();
    if (!live) return;
    uint8_t *out = y + sb * 84;
    out[g] = scb;
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int i = 4 * g + e, j = 128 * (i >> 5), l = i & 31;
        w |= (uint32_t)(Ls[sl][j + l] | (Ls[sl][j + l + 32] << 2) | (Ls[sl][j + l + 64] << 4) | (Ls[sl][j + l + 96] << 6)) << (8 * e);
    }
    *reinterpret_cast<uint32_t *>(out + 16 + 4 * g) = w;
    if (g == 0) *reinterpret_cast<uint32_t *>(out + 80) = (uint32_t)__half_as_ushort(dh) | ((uint32_t)__half_as_ushort(dmh) << 16);
}

// ------------------------------------------------------------------ Q3_K
// One thread per 16-element group. make_q3_quants(16, 4, x, L, true): codes -4..3 for weights x^2, then up to five passes
// that move one code at a time where that raises (sum w x l)^2 / (sum w l^2). Block {u8 hmask[32]; u8 qs[64];
// u8 scales[12] (sixteen 6-bit codes); f16 d} = 110 B.
__global__ void __launch_bounds__(256) k_quantize_q3_K(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nsuper) {
    __shared__ uint8_t Ls[16][256];
    __shared__ uint8_t sc6[16][16];
    const int tid = threadIdx.x, g = tid & 15, sl = tid >> 4;
    int64_t sb = (int64_t)blockIdx.x * 16 + sl;
    const bool live = sb < nsuper;
    if (!live) sb = nsuper - 1;
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 t = reinterpret_cast<const float4 *>(x + sb * 256 + g * 16)[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    int L[16];
    float scale = 0.f;
    {
        float mx = 0.f, amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (fabsf(v[i]) > amax) { amax = fabsf(v[i]); mx = v[i]; }
        if (amax < 1e-15f) {
#pragma unroll
            for (int i = 0; i < 16; i++) L[i] = 0;
        } else {
            const float iscale = __fdiv_rn(-4.f, mx);
            float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int l = max(-4, min(3, nearest_int(__fmul_rn(iscale, v[i]))));
                L[i] = l;
                const float w = __fmul_rn(v[i], v[i]);
                sumlx = __fadd_rn(sumlx, __fmul_rn(__fmul_rn(w, v[i]), (float)l));
                suml2 = __fadd_rn(suml2, __fmul_rn(__fmul_rn(w, (float)l), (float)l));
            }
            for (int itry = 0; itry < 5; itry++) {
                int changed = 0;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float w = __fmul_rn(v[i], v[i]);
                    float slx = __fsub_rn(sumlx, __fmul_rn(__fmul_rn(w, v[i]), (float)L[i]));
                    if (slx > 0.f) {
                        float sl2 = __fsub_rn(suml2, __fmul_rn(__fmul_rn(w, (float)L[i]), (float)L[i]));
                        const int nl = max(-4, min(3, nearest_int(__fdiv_rn(__fmul_rn(v[i], sl2), slx))));
                        if (nl != L[i]) {
                            slx = __fadd_rn(slx, __fmul_rn(__fmul_rn(w, v[i]), (float)nl));
                            sl2 = __fadd_rn(sl2, __fmul_rn(__fmul_rn(w, (float)nl), (float)nl));
                            if (sl2 > 0.f && __fmul_rn(__fmul_rn(slx, slx), suml2) > __fmul_rn(__fmul_rn(sumlx, sumlx), sl2)) {
                                L[i] = nl;
                                sumlx = slx;
                                suml2 = sl2;
                                changed++;
                            }
                        }
                    }
                }
                if (!changed) break;
            }
#pragma unroll
            for (int i = 0; i < 16; i++) L[i] += 4;
            scale = suml2 > 0.f ? __fdiv_rn(sumlx, suml2) : 0.f;
        }
    }
    const float max_scale = first_largest_magnitude16(scale, g);
    int l6 = 0;
    __half dh = __float2half_rn(0.f);
    if (max_scale != 0.f) {
        const float iscale = __fdiv_rn(-32.f, max_scale);
        const int l = (int)(signed char)nearest_int(__fmul_rn(iscale, scale));
        l6 = max(-32, min(31, l)) + 32;
        dh = __float2half_rn(__fdiv_rn(1.f, iscale));
    }
    const float d = __fmul_rn(__half2float(dh), (float)(l6 - 32));
    if (d != 0.f) {
#pragma unroll
        for (int i = 0; i < 16; i++) L[i] = max(-4, min(3, nearest_int(__fdiv_rn(v[i], d)))) + 4;
    }
#pragma unroll
    for (int i = 0; i < 16; i++) Ls[sl][g * 16 + i] = (uint8_t)L[i];
    sc6[sl][g] = (uint8_t)l6;
    __syncwarp();
    if (!live) return;
    uint8_t *out = y + sb * 110;
    // hmask[m], m in {2g, 2g+1}: bit b is the high bit of element 32b + m
    uint32_t hm = 0;
#pragma unroll
    for (int e = 0; e < 2; e++)
#pragma unroll
        for (int b = 0; b < 8; b++) hm |= (uint32_t)(Ls[sl][32 * b + 2 * g + e] >> 2) << (8 * e + b);
    *reinterpret_cast<uint16_t *>(out + 2 * g) = (uint16_t)hm;
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int i = 4 * g + e, j = 128 * (i >> 5), l = i & 31;
        w |= (uint32_t)((Ls[sl][j + l] & 3) | ((Ls[sl][j + l + 32] & 3) << 2) | ((Ls[sl][j + l + 64] & 3) << 4) | ((Ls[sl][j + l + 96] & 3) << 6)) << (8 * e);
    }
    *reinterpret_cast<uint16_t *>(out + 32 + 4 * g) = (uint16_t)(w & 0xffff);
    *reinterpret_cast<uint16_t *>(out + 32 + 4 * g + 2) = (uint16_t)(w >> 16);
    const uint8_t *s6 = sc6[sl];
    if (g < 8) out[96 + g] = (uint8_t)((s6[g] & 0xF) | ((s6[g + 8] & 0xF) << 4));
    else if (g < 12) {
        const int k = g - 8;
        out[96 + g] = (uint8_t)((s6[k] >> 4) | ((s6[k + 4] >> 4) << 2) | ((s6[k + 8] >> 4) << 4) | ((s6[k + 12] >> 4) << 6));
    } else if (g == 12) *reinterpret_cast<uint16_t *>(out + 108) = __half_as_ushort(dh);
}

// ------------------------------------------------------------------ Q6_K
// One thread per 16-element group. make_qx_quants(16, 32, x, L, 1, NULL): codes -32..31 for weights x^2, the scale tried at
// 18 more values around -32 / (value of largest magnitude). Block {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d} = 210 B.
__global__ void __launch_bounds__(256) k_quantize_q6_K(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                        int64_t nsuper) {
    __shared__ uint8_t Ls[16][256];
    const int tid = threadIdx.x, g = tid & 15, sl = tid >> 4;
    int64_t sb = (int64_t)blockIdx.x * 16 + sl;
    const bool live = sb < nsuper;
    if (!live) sb = nsuper - 1;
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 t = reinterpret_cast<const float4 *>(x + sb * 256 + g * 16)[i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    float mx = 0.f, amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++)
        if (fabsf(v[i]) > amax) { amax = fabsf(v[i]); mx = v[i]; }
    const bool zero = amax < 1e-15f;
    float scale = 0.f, win = 0.f;   // win: the iscale whose codes the search kept
    if (!zero) {
        float iscale = __fdiv_rn(-32.f, mx);
        float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float l = (float)max(-32, min(31, nearest_int(__fmul_rn(iscale, v[i]))));
            const float w = __fmul_rn(v[i], v[i]);
            sumlx = __fadd_rn(sumlx, __fmul_rn(__fmul_rn(w, v[i]), l));
            suml2 = __fadd_rn(suml2, __fmul_rn(__fmul_rn(w, l), l));
        }
        scale = suml2 != 0.f ? __fdiv_rn(sumlx, suml2) : 0.f;
        float best = __fmul_rn(scale, sumlx);
        win = iscale;
        for (int is = -9; is <= 9; is++) {
            if (is == 0) continue;
            iscale = __fdiv_rn(-__fadd_rn(32.f, __fmul_rn(0.1f, (float)is)), mx);
            sumlx = 0.f;
            suml2 = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float l = (float)max(-32, min(31, nearest_int(__fmul_rn(iscale, v[i]))));
                const float w = __fmul_rn(v[i], v[i]);
                sumlx = __fadd_rn(sumlx, __fmul_rn(__fmul_rn(w, v[i]), l));
                suml2 = __fadd_rn(suml2, __fmul_rn(__fmul_rn(w, l), l));
            }
            if (suml2 > 0.f && __fmul_rn(sumlx, sumlx) > __fmul_rn(best, suml2)) {
                win = iscale;
                scale = __fdiv_rn(sumlx, suml2);
                best = __fmul_rn(scale, sumlx);
            }
        }
    }
    const float max_scale = first_largest_magnitude16(scale, g);
    const bool dead = fabsf(max_scale) < 1e-15f;   // the whole super-block is written as zeros
    int sc = 0;
    __half dh = __float2half_rn(0.f);
    uint8_t *Lrow = &Ls[sl][g * 16];
    if (!dead) {
        const float iscale = __fdiv_rn(-128.f, max_scale);
        dh = __float2half_rn(__fdiv_rn(1.f, iscale));
        sc = (int)(signed char)min(127, nearest_int(__fmul_rn(iscale, scale)));
        const float d = __fmul_rn(__half2float(dh), (float)sc);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            int l;
            if (d != 0.f) l = max(-32, min(31, nearest_int(__fdiv_rn(v[i], d)))) + 32;
            else l = zero ? 0 : 32 + max(-32, min(31, nearest_int(__fmul_rn(win, v[i]))));
            Lrow[i] = (uint8_t)l;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) Lrow[i] = 0;
    }
    __syncwarp();
    if (!live) return;
    uint8_t *out = y + sb * 210;
    const uint8_t *Lb = Ls[sl];
    // ql[i], i in [8g, 8g+8): half h = i / 64 covers elements [128h, 128h+128)
    uint32_t q[2] = {0, 0};
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const int i = 8 * g + e, j = 128 * (i >> 6), r = i & 63, l = r & 31;
        const uint32_t byte = r < 32 ? (uint32_t)((Lb[j + l] & 0xF) | ((Lb[j + l + 64] & 0xF) << 4))
                                     : (uint32_t)((Lb[j + l + 32] & 0xF) | ((Lb[j + l + 96] & 0xF) << 4));
        q[e >> 2] |= byte << (8 * (e & 3));
    }
    uint16_t *o16 = reinterpret_cast<uint16_t *>(out);
    o16[4 * g] = (uint16_t)(q[0] & 0xffff);
    o16[4 * g + 1] = (uint16_t)(q[0] >> 16);
    o16[4 * g + 2] = (uint16_t)(q[1] & 0xffff);
    o16[4 * g + 3] = (uint16_t)(q[1] >> 16);
    uint32_t h = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int i = 4 * g + e, j = 128 * (i >> 5), l = i & 31;
        h |= (uint32_t)((Lb[j + l] >> 4) | ((Lb[j + l + 32] >> 4) << 2) | ((Lb[j + l + 64] >> 4) << 4) | ((Lb[j + l + 96] >> 4) << 6)) << (8 * e);
    }
    o16[64 + 2 * g] = (uint16_t)(h & 0xffff);
    o16[64 + 2 * g + 1] = (uint16_t)(h >> 16);
    out[192 + g] = dead ? 0 : (uint8_t)sc;
    if (g == 0) o16[104] = __half_as_ushort(dh);
}

// ------------------------------------------------------------------ F16 rows
__global__ void k_f32_to_f16(const float *__restrict__ x, __half *__restrict__ y, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(x[i]);
}

// round to nearest even on the upper 16 bits; a NaN stays a quiet NaN
__global__ void k_f32_to_bf16(const float *__restrict__ x, uint16_t *__restrict__ y, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t u = __float_as_uint(x[i]);
    y[i] = (u & 0x7fffffffu) > 0x7f800000u ? (uint16_t)((u >> 16) | 64) : (uint16_t)((u + (0x7fffu + ((u >> 16) & 1u))) >> 16);
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
            k_quantize_q45_K<false><<<(unsigned)((nb + 31) / 32), 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_Q5_K: {
            const int64_t nb = n / 256;
            k_quantize_q45_K<true><<<(unsigned)((nb + 31) / 32), 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_Q4_1: case TLB_TYPE_Q5_0: case TLB_TYPE_Q5_1: {
            const int64_t nb = n / 32;
            const unsigned grid = (unsigned)((nb * 8 + 255) / 256);
            if (type == TLB_TYPE_Q4_1) k_quantize_q451<0><<<grid, 256, 0, st>>>(x, (uint8_t *)y, nb);
            else if (type == TLB_TYPE_Q5_0) k_quantize_q451<1><<<grid, 256, 0, st>>>(x, (uint8_t *)y, nb);
            else k_quantize_q451<2><<<grid, 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_Q2_K: case TLB_TYPE_Q3_K: case TLB_TYPE_Q6_K: {
            const int64_t nb = n / 256;
            const unsigned grid = (unsigned)((nb + 15) / 16);
            if (type == TLB_TYPE_Q2_K) k_quantize_q2_K<<<grid, 256, 0, st>>>(x, (uint8_t *)y, nb);
            else if (type == TLB_TYPE_Q3_K) k_quantize_q3_K<<<grid, 256, 0, st>>>(x, (uint8_t *)y, nb);
            else k_quantize_q6_K<<<grid, 256, 0, st>>>(x, (uint8_t *)y, nb);
            break;
        }
        case TLB_TYPE_BF16:
            k_f32_to_bf16<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, (uint16_t *)y, n);
            break;
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
