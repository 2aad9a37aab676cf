/* TEST INFRASTRUCTURE ONLY -- see oracle.h. Compile with -ffp-contract=off (the reference's
 * build has no FMA contraction and the Q4_K scale search is sensitive to it). */
#include "oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- f16 <-> f32
 * IEEE binary16, round-to-nearest-even: what GGML_FP32_TO_FP16 / GGML_FP16_TO_FP32 compute
 * (vendor/ggml/src/ggml-impl.h:407-431). */
uint16_t orc_f32_to_f16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t mag = u & 0x7fffffffu;
    if (mag > 0x7f800000u) return (uint16_t)(sign | 0x7e00u); /* NaN */
    if (mag >= 0x47800000u) {                                  /* >= 65536: inf (65520.. rounds up below) */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (mag < 0x38800000u) { /* result is subnormal or zero: value * 2^24 rounded to an integer */
        if (mag < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to zero */
        int e = (int)(mag >> 23);
        uint32_t m = (mag & 0x7fffffu) | 0x800000u;
        int shift = 126 - e; /* m * 2^(e-150) * 2^24 = m >> (126 - e) */
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t e = (mag >> 23) - 112u;
    uint32_t m = mag & 0x7fffffu;
    uint32_t h = (e << 10) | (m >> 13);
    uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++; /* carries into the exponent correctly */
    return (uint16_t)(sign | h);
}

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) {
            u = sign;
        } else {
            int s = 0;
            while (!(m & 0x400u)) { m <<= 1; s++; }
            m &= 0x3ffu;
            u = sign | ((uint32_t)(113 - s) << 23) | (m << 13);
        }
    } else if (e == 31) {
        u = sign | 0x7f800000u | (m << 13);
    } else {
        u = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---------------------------------------------------------------- block layouts
 * vendor/ggml/src/ggml-common.h:194-199 (q4_0), :251-256 (q8_0), :327-338 (q4_K), :371-375 (q8_K) */
#pragma pack(push, 1)
typedef struct { uint16_t d; uint8_t qs[16]; } blk_q4_0;                       /* 18 B / 32  */
typedef struct { uint16_t d; int8_t qs[32]; } blk_q8_0;                        /* 34 B / 32  */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_K; /* 144 B / 256 */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_K;       /* 292 B / 256 */
typedef struct { uint16_t d, m; uint8_t qs[16]; } blk_q4_1;                    /* 20 B / 32  */
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_0;        /* 22 B / 32  */
typedef struct { uint16_t d, m; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_1;     /* 24 B / 32  */
typedef struct { uint8_t scales[16]; uint8_t qs[64]; uint16_t d, dmin; } blk_q2_K;                  /* 84 B / 256  */
typedef struct { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; } blk_q3_K;     /* 110 B / 256 */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; } blk_q5_K; /* 176 B / 256 */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6_K;        /* 210 B / 256 */
#pragma pack(pop)

int64_t orc_row_size(int type, int64_t ne0) {
    switch (type) {
        case ORC_F32: return ne0 * 4;
        case ORC_F16: return ne0 * 2;
        case ORC_BF16: return ne0 * 2;
        case ORC_Q4_0: return ne0 / 32 * 18;
        case ORC_Q8_0: return ne0 / 32 * 34;
        case ORC_Q4_K: return ne0 / 256 * 144;
        case ORC_Q4_1: return ne0 / 32 * 20;
        case ORC_Q5_0: return ne0 / 32 * 22;
        case ORC_Q5_1: return ne0 / 32 * 24;
        case ORC_Q2_K: return ne0 / 256 * 84;
        case ORC_Q3_K: return ne0 / 256 * 110;
        case ORC_Q5_K: return ne0 / 256 * 176;
        case ORC_Q6_K: return ne0 / 256 * 210;
        default: return -1;
    }
}

/* ggml-quants.c:621-626: round to nearest (ties to even) through the 1.5*2^23 magic constant */
static int near_int(float v) {
    float t = v + 12582912.f;
    int32_t i;
    memcpy(&i, &t, 4);
    return (i & 0x007fffff) - 0x00400000;
}

/* ggml-quants.c:276-299 */
void orc_quantize_row_q8_0(const float *x, void *vy, int64_t k) {
    blk_q8_0 *y = (blk_q8_0 *)vy;
    for (int64_t b = 0; b < k / 32; b++) {
        const float *xb = x + b * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; j++) {
            float a = fabsf(xb[j]);
            if (a > amax) amax = a;
        }
        const float d = amax / 127;
        const float id = d ? 1.0f / d : 0.0f;
        y[b].d = orc_f32_to_f16(d);
        for (int j = 0; j < 32; j++) y[b].qs[j] = (int8_t)roundf(xb[j] * id);
    }
}

/* ggml-quants.c:113-148 */
void orc_quantize_row_q4_0(const float *x, void *vy, int64_t k) {
    blk_q4_0 *y = (blk_q4_0 *)vy;
    for (int64_t b = 0; b < k / 32; b++) {
        const float *xb = x + b * 32;
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < 32; j++) {
            if (amax < fabsf(xb[j])) { amax = fabsf(xb[j]); max = xb[j]; }
        }
        const float d = max / -8;
        const float id = d ? 1.0f / d : 0.0f;
        y[b].d = orc_f32_to_f16(d);
        for (int j = 0; j < 16; j++) {
            const float x0 = xb[j] * id, x1 = xb[16 + j] * id;
            int a = (int8_t)(x0 + 8.5f), c = (int8_t)(x1 + 8.5f);
            uint8_t lo = (uint8_t)(a > 15 ? 15 : a), hi = (uint8_t)(c > 15 ? 15 : c);
            y[b].qs[j] = (uint8_t)(lo | (hi << 4));
        }
    }
}

/* ggml-quants.c:799-878 (make_qkx2_quants): weighted least-squares search of (scale, min) for codes 0..nmax.
 * Q4_K calls it with n=32, nmax=15, rmin=-1, nstep=20, squared error; Q5_K with nmax=31, rmin=-0.5, nstep=15;
 * Q2_K with n=16, nmax=3, rmin=-0.5, nstep=15 and the absolute error (use_mad). rdelta is 0.1 everywhere. */
static float search_scale_min(int n, int nmax, const float *x, const float *w, uint8_t *L, float *the_min, uint8_t *Laux,
                              float rmin, int nstep, int use_mad) {
    const float rdelta = 0.1f;
    float min = x[0], max = x[0];
    float sum_w = w[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; i++) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        sum_w += w[i];
        sum_x += w[i] * x[i];
    }
    if (min > 0) min = 0;
    if (max == min) {
        for (int i = 0; i < n; i++) L[i] = 0;
        *the_min = -min;
        return 0.f;
    }
    float iscale = nmax / (max - min);
    float scale = 1 / iscale;
    float best = 0;
    for (int i = 0; i < n; i++) {
        int l = near_int(iscale * (x[i] - min));
        l = l < 0 ? 0 : (l > nmax ? nmax : l);
        L[i] = (uint8_t)l;
        float diff = scale * L[i] + min - x[i];
        diff = use_mad ? fabsf(diff) : diff * diff;
        best += w[i] * diff;
    }
    for (int is = 0; is <= nstep; is++) {
        iscale = (rmin + rdelta * is + nmax) / (max - min);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < n; i++) {
            int l = near_int(iscale * (x[i] - min));
            l = l < 0 ? 0 : (l > nmax ? nmax : l);
            Laux[i] = (uint8_t)l;
            sum_l += w[i] * l;
            sum_l2 += w[i] * l * l;
            sum_xl += w[i] * l * x[i];
        }
        float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0) {
                this_min = 0;
                this_scale = sum_xl / sum_l2;
            }
            float err = 0;
            for (int i = 0; i < n; i++) {
                float diff = this_scale * Laux[i] + this_min - x[i];
                diff = use_mad ? fabsf(diff) : diff * diff;
                err += w[i] * diff;
            }
            if (err < best) {
                memcpy(L, Laux, (size_t)n);
                best = err;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

/* ggml-quants.c:880-887 */
static void scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ggml-quants.c:1457-1527 */
void orc_quantize_row_q4_K(const float *x, void *vy, int64_t k) {
    blk_q4_K *y = (blk_q4_K *)vy;
    uint8_t L[256], Laux[32];
    float weights[32], mins[8], scales[8];
    for (int64_t b = 0; b < k / 256; b++, x += 256) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 8; j++) {
            const float *xs = x + 32 * j;
            float sum_x2 = 0;
            for (int l = 0; l < 32; l++) sum_x2 += xs[l] * xs[l];
            float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; l++) weights[l] = av_x + fabsf(xs[l]);
            scales[j] = search_scale_min(32, 15, xs, weights, L + 32 * j, &mins[j], Laux, -1.f, 20, 0);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        memset(y[b].scales, 0, 12);
        for (int j = 0; j < 8; j++) {
            uint8_t ls = (uint8_t)near_int(inv_scale * scales[j]);
            uint8_t lm = (uint8_t)near_int(inv_min * mins[j]);
            if (ls > 63) ls = 63;
            if (lm > 63) lm = 63;
            if (j < 4) {
                y[b].scales[j] = ls;
                y[b].scales[j + 4] = lm;
            } else {
                y[b].scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                y[b].scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                y[b].scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        y[b].d = orc_f32_to_f16(max_scale / 63.f);
        y[b].dmin = orc_f32_to_f16(max_min / 63.f);
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            scale_min_k4(j, y[b].scales, &sc, &m);
            const float d = orc_f16_to_f32(y[b].d) * sc;
            if (!d) continue;
            const float dm = orc_f16_to_f32(y[b].dmin) * m;
            for (int i = 0; i < 32; i++) {
                int l = near_int((x[32 * j + i] + dm) / d);
                l = l < 0 ? 0 : (l > 15 ? 15 : l);
                L[32 * j + i] = (uint8_t)l;
            }
        }
        uint8_t *q = y[b].qs;
        for (int j = 0; j < 256; j += 64, q += 32)
            for (int l = 0; l < 32; l++) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
    }
}

/* ggml-quants.c:2768-2805 */
void orc_quantize_row_q8_K(const float *x, void *vy, int64_t k) {
    blk_q8_K *y = (blk_q8_K *)vy;
    for (int64_t b = 0; b < k / 256; b++, x += 256) {
        float max = 0, amax = 0;
        for (int j = 0; j < 256; j++) {
            float ax = fabsf(x[j]);
            if (ax > amax) { amax = ax; max = x[j]; }
        }
        if (!amax) {
            memset(&y[b], 0, sizeof(blk_q8_K)); /* the reference leaves bsums untouched; see note */
            continue;
        }
        const float iscale = -127.f / max;
        for (int j = 0; j < 256; j++) {
            int v = near_int(iscale * x[j]);
            y[b].qs[j] = (int8_t)(v > 127 ? 127 : v);
        }
        for (int j = 0; j < 16; j++) {
            int sum = 0;
            for (int i = 0; i < 16; i++) sum += y[b].qs[j * 16 + i];
            y[b].bsums[j] = (int16_t)sum;
        }
        y[b].d = 1 / iscale;
    }
}
/* note on the all-zero block: the reference sets d = 0 and qs = 0 and does not write bsums
 * (ggml-quants.c:2782-2787); with d = 0 the block contributes 0*bsums to every dot product, so the
 * result only differs if the stale bsums*0 were NaN/inf, which int16 cannot be. Byte comparisons
 * of Q8_K in tests exclude the bsums of such blocks. */

/* ggml-quants.c:150-185: d = (max - min) / 15, m = min, codes (int8)((x - min) / d + 0.5) capped at 15 */
void orc_quantize_row_q4_1(const float *x, void *vy, int64_t k) {
    blk_q4_1 *y = (blk_q4_1 *)vy;
    for (int64_t b = 0; b < k / 32; b++) {
        const float *xb = x + b * 32;
        float min = FLT_MAX, max = -FLT_MAX;
        for (int j = 0; j < 32; j++) {
            if (xb[j] < min) min = xb[j];
            if (xb[j] > max) max = xb[j];
        }
        const float d = (max - min) / 15;
        const float id = d ? 1.0f / d : 0.0f;
        y[b].d = orc_f32_to_f16(d);
        y[b].m = orc_f32_to_f16(min);
        for (int j = 0; j < 16; j++) {
            const float x0 = (xb[j] - min) * id, x1 = (xb[16 + j] - min) * id;
            const int a = (int8_t)(x0 + 0.5f), c = (int8_t)(x1 + 0.5f);
            const uint8_t lo = (uint8_t)(a > 15 ? 15 : a), hi = (uint8_t)(c > 15 ? 15 : c);
            y[b].qs[j] = (uint8_t)(lo | (hi << 4));
        }
    }
}

/* ggml-quants.c:187-229: d = (signed value of largest magnitude) / -16; the fifth bit of element e is bit e of qh */
void orc_quantize_row_q5_0(const float *x, void *vy, int64_t k) {
    blk_q5_0 *y = (blk_q5_0 *)vy;
    for (int64_t b = 0; b < k / 32; b++) {
        const float *xb = x + b * 32;
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < 32; j++)
            if (amax < fabsf(xb[j])) { amax = fabsf(xb[j]); max = xb[j]; }
        const float d = max / -16;
        const float id = d ? 1.0f / d : 0.0f;
        y[b].d = orc_f32_to_f16(d);
        uint32_t qh = 0;
        for (int j = 0; j < 16; j++) {
            const float x0 = xb[j] * id, x1 = xb[16 + j] * id;
            const int a = (int8_t)(x0 + 16.5f), c = (int8_t)(x1 + 16.5f);
            const uint8_t lo = (uint8_t)(a > 31 ? 31 : a), hi = (uint8_t)(c > 31 ? 31 : c);
            y[b].qs[j] = (uint8_t)((lo & 0x0F) | ((hi & 0x0F) << 4));
            qh |= (uint32_t)((lo & 0x10u) >> 4) << j;
            qh |= (uint32_t)((hi & 0x10u) >> 4) << (j + 16);
        }
        memcpy(y[b].qh, &qh, 4);
    }
}

/* ggml-quants.c:231-273: d = (max - min) / 31, m = min, codes (uint8)((x - min) / d + 0.5), no cap */
void orc_quantize_row_q5_1(const float *x, void *vy, int64_t k) {
    blk_q5_1 *y = (blk_q5_1 *)vy;
    for (int64_t b = 0; b < k / 32; b++) {
        const float *xb = x + b * 32;
        float min = FLT_MAX, max = -FLT_MAX;
        for (int j = 0; j < 32; j++) {
            if (xb[j] < min) min = xb[j];
            if (xb[j] > max) max = xb[j];
        }
        const float d = (max - min) / 31;
        const float id = d ? 1.0f / d : 0.0f;
        y[b].d = orc_f32_to_f16(d);
        y[b].m = orc_f32_to_f16(min);
        uint32_t qh = 0;
        for (int j = 0; j < 16; j++) {
            const float x0 = (xb[j] - min) * id, x1 = (xb[16 + j] - min) * id;
            const uint8_t lo = (uint8_t)(x0 + 0.5f), hi = (uint8_t)(x1 + 0.5f);
            y[b].qs[j] = (uint8_t)((lo & 0x0F) | ((hi & 0x0F) << 4));
            qh |= (uint32_t)((lo & 0x10u) >> 4) << j;
            qh |= (uint32_t)((hi & 0x10u) >> 4) << (j + 16);
        }
        memcpy(y[b].qh, &qh, 4);
    }
}

/* ggml-quants.c:891-958: 16 groups of 16 with 4-bit scale and 4-bit min each (one byte), 2-bit codes */
void orc_quantize_row_q2_K(const float *x, void *vy, int64_t k) {
    blk_q2_K *y = (blk_q2_K *)vy;
    uint8_t L[256], Laux[16];
    float weights[16], mins[16], scales[16];
    for (int64_t b = 0; b < k / 256; b++, x += 256) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 16; j++) {
            for (int l = 0; l < 16; l++) weights[l] = fabsf(x[16 * j + l]);
            scales[j] = search_scale_min(16, 3, x + 16 * j, weights, L + 16 * j, &mins[j], Laux, -0.5f, 15, 1);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        if (max_scale > 0) {
            const float iscale = 15.f / max_scale;
            for (int j = 0; j < 16; j++) y[b].scales[j] = (uint8_t)near_int(iscale * scales[j]);
            y[b].d = orc_f32_to_f16(max_scale / 15.f);
        } else {
            memset(y[b].scales, 0, 16);
            y[b].d = orc_f32_to_f16(0.f);
        }
        if (max_min > 0) {
            const float iscale = 15.f / max_min;
            for (int j = 0; j < 16; j++) y[b].scales[j] |= (uint8_t)(near_int(iscale * mins[j]) << 4);
            y[b].dmin = orc_f32_to_f16(max_min / 15.f);
        } else {
            y[b].dmin = orc_f32_to_f16(0.f);
        }
        for (int j = 0; j < 16; j++) {
            const float d = orc_f16_to_f32(y[b].d) * (y[b].scales[j] & 0xF);
            if (!d) continue;
            const float dm = orc_f16_to_f32(y[b].dmin) * (y[b].scales[j] >> 4);
            for (int i = 0; i < 16; i++) {
                int l = near_int((x[16 * j + i] + dm) / d);
                L[16 * j + i] = (uint8_t)(l < 0 ? 0 : (l > 3 ? 3 : l));
            }
        }
        for (int j = 0; j < 256; j += 128)
            for (int l = 0; l < 32; l++)
                y[b].qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

/* ggml-quants.c:697-754 (make_q3_quants, do_rmse): codes -nmax..nmax-1 for weights x^2, then up to five passes that move
 * one code at a time when that raises (sum w x l)^2 / (sum w l^2); returns the least-squares scale, codes stored + nmax */
static float search_scale_refine(int n, int nmax, const float *x, int8_t *L) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; i++) {
        float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < 1e-15f) {
        memset(L, 0, (size_t)n);
        return 0.f;
    }
    const float iscale = -nmax / max;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; i++) {
        int l = near_int(iscale * x[i]);
        l = l < -nmax ? -nmax : (l > nmax - 1 ? nmax - 1 : l);
        L[i] = (int8_t)l;
        const float w = x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    for (int itry = 0; itry < 5; itry++) {
        int changed = 0;
        for (int i = 0; i < n; i++) {
            const float w = x[i] * x[i];
            float slx = sumlx - w * x[i] * L[i];
            if (slx > 0) {
                float sl2 = suml2 - w * L[i] * L[i];
                int nl = near_int(x[i] * sl2 / slx);
                nl = nl < -nmax ? -nmax : (nl > nmax - 1 ? nmax - 1 : nl);
                if (nl != L[i]) {
                    slx += w * x[i] * nl;
                    sl2 += w * nl * nl;
                    if (sl2 > 0 && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        L[i] = (int8_t)nl;
                        sumlx = slx;
                        suml2 = sl2;
                        changed++;
                    }
                }
            }
        }
        if (!changed) break;
    }
    for (int i = 0; i < n; i++) L[i] = (int8_t)(L[i] + nmax);
    return suml2 > 0.0f ? sumlx / suml2 : 0.0f;
}

/* ggml-quants.c:1229-1303: 16 groups of 16, 6-bit signed group scales against d = max_scale / -32, 3-bit codes whose
 * high bit goes to hmask (bit j/32 of byte j%32) */
void orc_quantize_row_q3_K(const float *x, void *vy, int64_t k) {
    blk_q3_K *y = (blk_q3_K *)vy;
    int8_t L[256];
    float scales[16];
    for (int64_t b = 0; b < k / 256; b++, x += 256) {
        float max_scale = 0, amax = 0;
        for (int j = 0; j < 16; j++) {
            scales[j] = search_scale_refine(16, 4, x + 16 * j, L + 16 * j);
            const float a = fabsf(scales[j]);
            if (a > amax) { amax = a; max_scale = scales[j]; }
        }
        memset(y[b].scales, 0, 12);
        if (max_scale) {
            const float iscale = -32.f / max_scale;
            for (int j = 0; j < 16; j++) {
                int8_t l = (int8_t)near_int(iscale * scales[j]);
                l = (int8_t)((l < -32 ? -32 : (l > 31 ? 31 : l)) + 32);
                if (j < 8) y[b].scales[j] = (uint8_t)(l & 0xF);
                else y[b].scales[j - 8] |= (uint8_t)((l & 0xF) << 4);
                l >>= 4;
                y[b].scales[j % 4 + 8] |= (uint8_t)(l << (2 * (j / 4)));
            }
            y[b].d = orc_f32_to_f16(1 / iscale);
        } else {
            y[b].d = orc_f32_to_f16(0.f);
        }
        for (int j = 0; j < 16; j++) {
            int8_t sc = (int8_t)(j < 8 ? y[b].scales[j] & 0xF : y[b].scales[j - 8] >> 4);
            sc = (int8_t)((sc | (((y[b].scales[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32);
            const float d = orc_f16_to_f32(y[b].d) * sc;
            if (!d) continue;
            for (int i = 0; i < 16; i++) {
                int l = near_int(x[16 * j + i] / d);
                l = l < -4 ? -4 : (l > 3 ? 3 : l);
                L[16 * j + i] = (int8_t)(l + 4);
            }
        }
        memset(y[b].hmask, 0, 32);
        for (int j = 0; j < 256; j++)
            if (L[j] > 3) {
                y[b].hmask[j % 32] |= (uint8_t)(1 << (j / 32));
                L[j] = (int8_t)(L[j] - 4);
            }
        for (int j = 0; j < 256; j += 128)
            for (int l = 0; l < 32; l++)
                y[b].qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
    }
}

/* ggml-quants.c:1644-1727: Q4_K's scheme with 5-bit codes (search with nmax 31, rmin -0.5, 15 steps); bit 2c / 2c+1 of
 * qh[j] is the fifth bit of element 64c + j / 64c + 32 + j */
void orc_quantize_row_q5_K(const float *x, void *vy, int64_t k) {
    blk_q5_K *y = (blk_q5_K *)vy;
    uint8_t L[256], Laux[32];
    float weights[32], mins[8], scales[8];
    for (int64_t b = 0; b < k / 256; b++, x += 256) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 8; j++) {
            const float *xs = x + 32 * j;
            float sum_x2 = 0;
            for (int l = 0; l < 32; l++) sum_x2 += xs[l] * xs[l];
            const float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; l++) weights[l] = av_x + fabsf(xs[l]);
            scales[j] = search_scale_min(32, 31, xs, weights, L + 32 * j, &mins[j], Laux, -0.5f, 15, 0);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        const float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        const float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        memset(y[b].scales, 0, 12);
        for (int j = 0; j < 8; j++) {
            uint8_t ls = (uint8_t)near_int(inv_scale * scales[j]);
            uint8_t lm = (uint8_t)near_int(inv_min * mins[j]);
            if (ls > 63) ls = 63;
            if (lm > 63) lm = 63;
            if (j < 4) {
                y[b].scales[j] = ls;
                y[b].scales[j + 4] = lm;
            } else {
                y[b].scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                y[b].scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                y[b].scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        y[b].d = orc_f32_to_f16(max_scale / 63.f);
        y[b].dmin = orc_f32_to_f16(max_min / 63.f);
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            scale_min_k4(j, y[b].scales, &sc, &m);
            const float d = orc_f16_to_f32(y[b].d) * sc;
            if (!d) continue;
            const float dm = orc_f16_to_f32(y[b].dmin) * m;
            for (int i = 0; i < 32; i++) {
                int l = near_int((x[32 * j + i] + dm) / d);
                L[32 * j + i] = (uint8_t)(l < 0 ? 0 : (l > 31 ? 31 : l));
            }
        }
        memset(y[b].qh, 0, 32);
        uint8_t *ql = y[b].qs;
        for (int n = 0, c = 0; n < 256; n += 64, c++, ql += 32)
            for (int j = 0; j < 32; j++) {
                int l1 = L[n + j], l2 = L[n + j + 32];
                if (l1 > 15) { l1 -= 16; y[b].qh[j] |= (uint8_t)(1 << (2 * c)); }
                if (l2 > 15) { l2 -= 16; y[b].qh[j] |= (uint8_t)(2 << (2 * c)); }
                ql[j] = (uint8_t)(l1 | (l2 << 4));
            }
    }
}

/* ggml-quants.c:628-695 (make_qx_quants with rmse_type 1, no external weights): codes -nmax..nmax-1 stored + nmax, weights
 * x^2, the scale tried at 18 more values around -nmax / (value of largest magnitude) */
static float search_scale_sym(int n, int nmax, const float *x, int8_t *L) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; i++) {
        float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < 1e-15f) {
        memset(L, 0, (size_t)n);
        return 0.f;
    }
    float iscale = -nmax / max;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; i++) {
        int l = near_int(iscale * x[i]);
        l = l < -nmax ? -nmax : (l > nmax - 1 ? nmax - 1 : l);
        L[i] = (int8_t)(l + nmax);
        const float w = x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; is++) {
        if (is == 0) continue;
        iscale = -(nmax + 0.1f * is) / max;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; i++) {
            int l = near_int(iscale * x[i]);
            l = l < -nmax ? -nmax : (l > nmax - 1 ? nmax - 1 : l);
            const float w = x[i] * x[i];
            sumlx += w * x[i] * l;
            suml2 += w * l * l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; i++) {
                int l = near_int(iscale * x[i]);
                l = l < -nmax ? -nmax : (l > nmax - 1 ? nmax - 1 : l);
                L[i] = (int8_t)(nmax + l);
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

/* ggml-quants.c:1869-1937: 16 groups of 16, int8 group scales against d = max_scale / -128, 6-bit codes split into
 * ql (low nibbles) and qh (high two bits) */
void orc_quantize_row_q6_K(const float *x, void *vy, int64_t k) {
    blk_q6_K *y = (blk_q6_K *)vy;
    int8_t L[256];
    float scales[16];
    for (int64_t b = 0; b < k / 256; b++, x += 256) {
        float max_scale = 0, max_abs_scale = 0;
        for (int j = 0; j < 16; j++) {
            scales[j] = search_scale_sym(16, 32, x + 16 * j, L + 16 * j);
            const float a = fabsf(scales[j]);
            if (a > max_abs_scale) { max_abs_scale = a; max_scale = scales[j]; }
        }
        if (max_abs_scale < 1e-15f) {
            memset(&y[b], 0, sizeof(blk_q6_K));
            continue;
        }
        const float iscale = -128.f / max_scale;
        y[b].d = orc_f32_to_f16(1 / iscale);
        for (int j = 0; j < 16; j++) {
            const int l = near_int(iscale * scales[j]);
            y[b].scales[j] = (int8_t)(l > 127 ? 127 : l);
        }
        for (int j = 0; j < 16; j++) {
            const float d = orc_f16_to_f32(y[b].d) * y[b].scales[j];
            if (!d) continue;
            for (int i = 0; i < 16; i++) {
                int l = near_int(x[16 * j + i] / d);
                l = l < -32 ? -32 : (l > 31 ? 31 : l);
                L[16 * j + i] = (int8_t)(l + 32);
            }
        }
        uint8_t *ql = y[b].ql, *qh = y[b].qh;
        for (int j = 0; j < 256; j += 128, ql += 64, qh += 32)
            for (int l = 0; l < 32; l++) {
                const uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF, q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
                ql[l] = (uint8_t)(q1 | (q3 << 4));
                ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
                qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
            }
    }
}

/* ggml-impl.h ggml_compute_fp32_to_bf16: round to nearest even on the upper 16 bits, NaN kept quiet */
static uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffff) > 0x7f800000) return (uint16_t)((u >> 16) | 64);
    return (uint16_t)((u + (0x7fff + ((u >> 16) & 1))) >> 16);
}

int orc_quantize_rows(int type, const float *src, int64_t nrows, int64_t n, void *dst) {
    int64_t rs = orc_row_size(type, n);
    if (rs < 0) return -1;
    for (int64_t r = 0; r < nrows; r++) {
        void *o = (char *)dst + r * rs;
        const float *s = src + r * n;
        switch (type) {
            case ORC_Q8_0: orc_quantize_row_q8_0(s, o, n); break;
            case ORC_Q4_0: orc_quantize_row_q4_0(s, o, n); break;
            case ORC_Q4_K: orc_quantize_row_q4_K(s, o, n); break;
            case ORC_Q4_1: orc_quantize_row_q4_1(s, o, n); break;
            case ORC_Q5_0: orc_quantize_row_q5_0(s, o, n); break;
            case ORC_Q5_1: orc_quantize_row_q5_1(s, o, n); break;
            case ORC_Q2_K: orc_quantize_row_q2_K(s, o, n); break;
            case ORC_Q3_K: orc_quantize_row_q3_K(s, o, n); break;
            case ORC_Q5_K: orc_quantize_row_q5_K(s, o, n); break;
            case ORC_Q6_K: orc_quantize_row_q6_K(s, o, n); break;
            case ORC_BF16: for (int64_t i = 0; i < n; i++) ((uint16_t *)o)[i] = f32_to_bf16(s[i]); break;
            case ORC_F16: for (int64_t i = 0; i < n; i++) ((uint16_t *)o)[i] = orc_f32_to_f16(s[i]); break;
            case ORC_F32: memcpy(o, s, (size_t)n * 4); break;
            default: return -1;
        }
    }
    return 0;
}

/* Element e of one block of the other block types, decoded the way ggml-quants.c does it row by row
 * (dequantize_row_q4_1 :479, _q5_0 :500, _q5_1 :526, _q2_K :961, _q3_K :1305, _q5_K :1731, _q6_K :1939; block layouts
 * ggml-common.h): every product and sum is a separate f32 operation, in ggml's order. */
static float f16_at(const uint8_t *p) { return orc_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }
static float decode_elem(int type, const uint8_t *b, int e) {
    switch (type) {
        case ORC_Q4_1: {  /* {f16 d, m; u8 qs[16]} */
            const int q = e < 16 ? (b[4 + e] & 0x0F) : (b[4 + e - 16] >> 4);
            const float t = (float)q * f16_at(b);
            return t + f16_at(b + 2);
        }
        case ORC_Q5_0: case ORC_Q5_1: {  /* {f16 d[, m]; u8 qh[4]; u8 qs[16]}: bit e of qh is the fifth bit of element e */
            const int one = type == ORC_Q5_1;
            const uint8_t *hb = b + (one ? 4 : 2), *qs = hb + 4;
            const uint32_t qh = (uint32_t)hb[0] | ((uint32_t)hb[1] << 8) | ((uint32_t)hb[2] << 16) | ((uint32_t)hb[3] << 24);
            const int q = (e < 16 ? (qs[e] & 0x0F) : (qs[e - 16] >> 4)) | (int)(((qh >> e) & 1u) << 4);
            if (one) { const float t = (float)q * f16_at(b); return t + f16_at(b + 2); }
            return (float)(q - 16) * f16_at(b);
        }
        case ORC_Q2_K: {  /* {u8 scales[16]; u8 qs[64]; f16 d, dmin} */
            const int n = e >> 7, j = (e >> 5) & 3, sub = (e >> 4) & 1, l = e & 15;
            const uint8_t sc = b[n * 8 + 2 * j + sub];
            const int q = (b[16 + n * 32 + sub * 16 + l] >> (2 * j)) & 3;
            const float dl = f16_at(b + 80) * (float)(sc & 0xF), ml = f16_at(b + 82) * (float)(sc >> 4);
            const float t = dl * (float)q;
            return t - ml;
        }
        case ORC_Q3_K: {  /* {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d} */
            const int n = e >> 7, j = (e >> 5) & 3, sub = (e >> 4) & 1, l = e & 15;
            const int is = n * 8 + 2 * j + sub, g = is >> 2, i = is & 3;
            const uint8_t *s = b + 96;
            const int lo = g < 2 ? (s[4 * g + i] & 0xF) : (s[4 * (g - 2) + i] >> 4);
            const int hi = (s[8 + i] >> (2 * g)) & 3;
            const int scale = (int)(int8_t)(lo | (hi << 4)) - 32;
            const int q = ((b[32 + n * 32 + sub * 16 + l] >> (2 * j)) & 3) - ((b[sub * 16 + l] & (1 << (4 * n + j))) ? 0 : 4);
            const float dl = f16_at(b + 108) * (float)scale;
            return dl * (float)q;
        }
        case ORC_Q5_K: {  /* {f16 d, dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} */
            const int j = e >> 5, l = e & 31;
            uint8_t sc, m;
            scale_min_k4(j, b + 4, &sc, &m);
            const int q = ((b[48 + (j >> 1) * 32 + l] >> ((j & 1) * 4)) & 0xF) + ((b[16 + l] & (1 << j)) ? 16 : 0);
            const float d1 = f16_at(b) * (float)sc, m1 = f16_at(b + 2) * (float)m;
            const float t = d1 * (float)q;
            return t - m1;
        }
        case ORC_Q6_K: {  /* {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d} */
            const int n = e >> 7, quarter = (e >> 5) & 3, l = e & 31;
            const uint8_t lo = b[n * 64 + (quarter & 1) * 32 + l];
            const int q = (int)(int8_t)(((quarter & 2) ? (lo >> 4) : (lo & 0xF)) | (((b[128 + n * 32 + l] >> (2 * quarter)) & 3) << 4)) - 32;
            const float ds = f16_at(b + 208) * (float)((const int8_t *)(b + 192))[n * 8 + (l >> 4) + 2 * quarter];
            return ds * (float)q;
        }
        default: return 0.f;
    }
}

/* ggml-quants.c dequantize_row_q8_0 / _q4_0 / _q4_K (:1529-1551) */
int orc_dequantize_row(int type, const void *src, float *y, int64_t k) {
    switch (type) {
        case ORC_Q4_1: case ORC_Q5_0: case ORC_Q5_1: case ORC_Q2_K: case ORC_Q3_K: case ORC_Q5_K: case ORC_Q6_K: {
            const int blck = (type == ORC_Q4_1 || type == ORC_Q5_0 || type == ORC_Q5_1) ? 32 : 256;
            const int64_t bytes = orc_row_size(type, blck);
            for (int64_t i = 0; i < k; i++) y[i] = decode_elem(type, (const uint8_t *)src + (i / blck) * bytes, (int)(i % blck));
            return 0;
        }
        case ORC_F32: memcpy(y, src, (size_t)k * 4); return 0;
        case ORC_F16: for (int64_t i = 0; i < k; i++) y[i] = orc_f16_to_f32(((const uint16_t *)src)[i]); return 0;
        case ORC_Q8_0: {
            const blk_q8_0 *x = (const blk_q8_0 *)src;
            for (int64_t b = 0; b < k / 32; b++) {
                const float d = orc_f16_to_f32(x[b].d);
                for (int j = 0; j < 32; j++) y[b * 32 + j] = x[b].qs[j] * d;
            }
            return 0;
        }
        case ORC_Q4_0: {
            const blk_q4_0 *x = (const blk_q4_0 *)src;
            for (int64_t b = 0; b < k / 32; b++) {
                const float d = orc_f16_to_f32(x[b].d);
                for (int j = 0; j < 16; j++) {
                    y[b * 32 + j] = ((x[b].qs[j] & 0x0F) - 8) * d;
                    y[b * 32 + j + 16] = ((x[b].qs[j] >> 4) - 8) * d;
                }
            }
            return 0;
        }
        case ORC_Q4_K: {
            const blk_q4_K *x = (const blk_q4_K *)src;
            for (int64_t b = 0; b < k / 256; b++) {
                const float d = orc_f16_to_f32(x[b].d), mn = orc_f16_to_f32(x[b].dmin);
                const uint8_t *q = x[b].qs;
                for (int j = 0; j < 4; j++, q += 32) {
                    uint8_t sc, m;
                    scale_min_k4(2 * j, x[b].scales, &sc, &m);
                    const float d1 = d * sc, m1 = mn * m;
                    scale_min_k4(2 * j + 1, x[b].scales, &sc, &m);
                    const float d2 = d * sc, m2 = mn * m;
                    for (int l = 0; l < 32; l++) *y++ = d1 * (q[l] & 0xF) - m1;
                    for (int l = 0; l < 32; l++) *y++ = d2 * (q[l] >> 4) - m2;
                }
            }
            return 0;
        }
        default: return -1;
    }
}

/* ---------------------------------------------------------------- dot products
 * generic (non-SIMD) versions: the ones the reference's -O3 build without -march runs */

/* ggml-cpu/quants.c:451-479 */
static float dot_q8_0_q8_0(int64_t n, const blk_q8_0 *x, const blk_q8_0 *y) {
    float sumf = 0;
    for (int64_t b = 0; b < n / 32; b++) {
        int sumi = 0;
        for (int j = 0; j < 32; j++) sumi += x[b].qs[j] * y[b].qs[j];
        sumf += sumi * (orc_f16_to_f32(x[b].d) * orc_f16_to_f32(y[b].d));
    }
    return sumf;
}

/* ggml-cpu/quants.c:225-260 */
static float dot_q4_0_q8_0(int64_t n, const blk_q4_0 *x, const blk_q8_0 *y) {
    float sumf = 0;
    for (int64_t b = 0; b < n / 32; b++) {
        int s0 = 0, s1 = 0;
        for (int j = 0; j < 16; j++) {
            const int v0 = (x[b].qs[j] & 0x0F) - 8, v1 = (x[b].qs[j] >> 4) - 8;
            s0 += v0 * y[b].qs[j];
            s1 += v1 * y[b].qs[j + 16];
        }
        int sumi = s0 + s1;
        sumf += sumi * orc_f16_to_f32(x[b].d) * orc_f16_to_f32(y[b].d);
    }
    return sumf;
}

/* ggml-cpu/quants.c:696-770 */
static float dot_q4_K_q8_K(int64_t n, const blk_q4_K *x, const blk_q8_K *y) {
    float sums[8] = {0};
    float sumf = 0;
    for (int64_t b = 0; b < n / 256; b++) {
        int8_t a[256];
        const uint8_t *q4 = x[b].qs;
        for (int j = 0; j < 4; j++, q4 += 32) {
            for (int l = 0; l < 32; l++) a[64 * j + l] = (int8_t)(q4[l] & 0xF);
            for (int l = 0; l < 32; l++) a[64 * j + 32 + l] = (int8_t)(q4[l] >> 4);
        }
        int32_t aux32[8] = {0};
        int sumi = 0;
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            scale_min_k4(j, x[b].scales, &sc, &m);
            sumi += (y[b].bsums[2 * j] + y[b].bsums[2 * j + 1]) * m;
            for (int g = 0; g < 4; g++)
                for (int l = 0; l < 8; l++) {
                    int i = 32 * j + 8 * g + l;
                    aux32[l] += (int32_t)sc * (int16_t)(y[b].qs[i] * a[i]);
                }
        }
        const float d = orc_f16_to_f32(x[b].d) * y[b].d;
        for (int l = 0; l < 8; l++) sums[l] += d * aux32[l];
        const float dmin = orc_f16_to_f32(x[b].dmin) * y[b].d;
        sumf -= dmin * sumi;
    }
    for (int l = 0; l < 8; l++) sumf += sums[l];
    return sumf;
}

/* ggml-cpu.c:1272-1357: src1 rows are converted with the weight type's vec_dot_type quantizer,
 * then every output is one vec_dot over the whole row. */
int orc_mul_mat(int type, const void *W, int64_t K, int64_t M, const float *x, int64_t N, float *y) {
    const int64_t wrow = orc_row_size(type, K);
    if (wrow < 0) return -1;
    if (type == ORC_F32 || type == ORC_F16) {
        float *row = (float *)malloc((size_t)K * 4);
        for (int64_t m = 0; m < M; m++) {
            orc_dequantize_row(type, (const char *)W + m * wrow, row, K);
            for (int64_t n = 0; n < N; n++) {
                double s = 0;
                for (int64_t k = 0; k < K; k++) s += (double)row[k] * (double)x[n * K + k];
                y[n * M + m] = (float)s;
            }
        }
        free(row);
        return 0;
    }
    const int kq = type == ORC_Q4_K;
    const int64_t arow = kq ? K / 256 * (int64_t)sizeof(blk_q8_K) : K / 32 * (int64_t)sizeof(blk_q8_0);
    char *act = (char *)malloc((size_t)(arow * N));
    for (int64_t n = 0; n < N; n++) {
        if (kq) orc_quantize_row_q8_K(x + n * K, act + n * arow, K);
        else orc_quantize_row_q8_0(x + n * K, act + n * arow, K);
    }
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            const void *w = (const char *)W + m * wrow;
            const void *a = act + n * arow;
            float r;
            if (type == ORC_Q8_0) r = dot_q8_0_q8_0(K, (const blk_q8_0 *)w, (const blk_q8_0 *)a);
            else if (type == ORC_Q4_0) r = dot_q4_0_q8_0(K, (const blk_q4_0 *)w, (const blk_q8_0 *)a);
            else r = dot_q4_K_q8_K(K, (const blk_q4_K *)w, (const blk_q8_K *)a);
            y[n * M + m] = r;
        }
    free(act);
    return 0;
}

int orc_mul_mat_dequant(int type, const void *W, int64_t K, int64_t M, const float *x, int64_t N, float *y) {
    const int64_t wrow = orc_row_size(type, K);
    if (wrow < 0) return -1;
    float *row = (float *)malloc((size_t)K * 4);
    for (int64_t m = 0; m < M; m++) {
        if (orc_dequantize_row(type, (const char *)W + m * wrow, row, K)) { free(row); return -1; }
        for (int64_t n = 0; n < N; n++) {
            double s = 0;
            for (int64_t k = 0; k < K; k++) s += (double)row[k] * (double)x[n * K + k];
            y[n * M + m] = (float)s;
        }
    }
    free(row);
    return 0;
}

/* ---------------------------------------------------------------- row ops */

/* ops.cpp:3794-3860: sum of squares in double, mean and scale in float */
void orc_rms_norm(const float *x, int64_t n, int64_t rows, float eps, const float *w, float *y) {
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * n;
        double sum = 0.0;
        for (int64_t i = 0; i < n; i++) sum += (double)(xr[i] * xr[i]);
        const float mean = (float)(sum / n);
        const float scale = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < n; i++) y[r * n + i] = w ? xr[i] * scale * w[i] : xr[i] * scale;
    }
}

void orc_silu_mul(const float *g, const float *u, int64_t n, float *y) {
    for (int64_t i = 0; i < n; i++) y[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
}

/* ops.cpp:5846-5860 (cache: theta multiplied up sequentially), :5935-5949 (pair rotation),
 * :6085-6093 (dims past n_dims copied). ext_factor = 0, no frequency factors. */
void orc_rope(const float *x, int64_t ne0, int64_t heads, int64_t tokens, const int32_t *pos, int n_dims,
              int mode, float freq_base, float freq_scale, float attn_factor, float *y) {
    const float theta_scale = powf(freq_base, -2.0f / n_dims);
    float *cache = (float *)malloc((size_t)ne0 * 4);
    for (int64_t t = 0; t < tokens; t++) {
        float theta = (float)pos[t];
        for (int64_t i0 = 0; i0 < ne0; i0 += 2) {
            const float th = freq_scale * theta;
            cache[i0] = cosf(th) * attn_factor;
            cache[i0 + 1] = sinf(th) * attn_factor;
            theta *= theta_scale;
        }
        for (int64_t h = 0; h < heads; h++) {
            const float *s = x + (t * heads + h) * ne0;
            float *d = y + (t * heads + h) * ne0;
            const int64_t off = mode == 0 ? 1 : n_dims / 2;
            for (int64_t i0 = 0; i0 < n_dims; i0 += 2) {
                const int64_t ic = mode == 0 ? i0 : i0 / 2;
                const float c = cache[i0], sn = cache[i0 + 1];
                const float x0 = s[ic], x1 = s[ic + off];
                d[ic] = x0 * c - x1 * sn;
                d[ic + off] = x0 * sn + x1 * c;
            }
            for (int64_t i0 = n_dims; i0 < ne0; i0++) d[i0] = s[i0];
        }
    }
    free(cache);
}

/* ops.cpp:5517-5554 with no mask: y = exp(x*scale - max) / sum (sum in double) */
void orc_soft_max(const float *x, int64_t n, int64_t rows, float scale, float *y) {
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * n;
        float *yr = y + r * n;
        float mx = -INFINITY;
        for (int64_t i = 0; i < n; i++) {
            yr[i] = xr[i] * scale;
            if (yr[i] > mx) mx = yr[i];
        }
        double sum = 0.0;
        for (int64_t i = 0; i < n; i++) {
            yr[i] = expf(yr[i] - mx);
            sum += (double)yr[i];
        }
        const float inv = (float)(1.0 / sum);
        for (int64_t i = 0; i < n; i++) yr[i] *= inv;
    }
}

int orc_get_rows(int type, const void *table, int64_t ne0, const int32_t *ids, int64_t n_ids, float *y) {
    const int64_t rs = orc_row_size(type, ne0);
    if (rs < 0) return -1;
    for (int64_t i = 0; i < n_ids; i++)
        if (orc_dequantize_row(type, (const char *)table + (int64_t)ids[i] * rs, y + i * ne0, ne0)) return -1;
    return 0;
}

void orc_argmax(const float *x, int64_t n, int64_t rows, int32_t *out) {
    for (int64_t r = 0; r < rows; r++) {
        float mx = -INFINITY;
        int32_t idx = 0;
        for (int64_t i = 0; i < n; i++) {
            if (x[r * n + i] > mx) mx = x[r * n + i];
            if (mx == x[r * n + i]) idx = (int32_t)i;
        }
        out[r] = idx;
    }
}

void orc_attention_decode(const uint16_t *q, const uint16_t *const *k, const uint16_t *const *v,
                          const int32_t *ctx, int seqs, int heads, int kv_heads, int hs, float scale,
                          uint16_t *out, float *out_f32) {
    const int group = heads / kv_heads;
    for (int s = 0; s < seqs; s++) {
        const int n = ctx[s];
        float *logit = (float *)malloc((size_t)(n > 0 ? n : 1) * 4);
        double *acc = (double *)malloc((size_t)hs * 8);
        for (int h = 0; h < heads; h++) {
            const int kvh = h / group;
            const uint16_t *qv = q + ((int64_t)s * heads + h) * hs;
            float mx = -INFINITY;
            for (int t = 0; t < n; t++) {
                const uint16_t *kr = k[s] + ((int64_t)t * kv_heads + kvh) * hs;
                double d = 0;
                for (int i = 0; i < hs; i++) d += (double)orc_f16_to_f32(qv[i]) * (double)orc_f16_to_f32(kr[i]);
                logit[t] = (float)d * scale;
                if (logit[t] > mx) mx = logit[t];
            }
            double sum = 0;
            for (int i = 0; i < hs; i++) acc[i] = 0;
            for (int t = 0; t < n; t++) {
                const double p = exp((double)logit[t] - (double)mx);
                sum += p;
                const uint16_t *vr = v[s] + ((int64_t)t * kv_heads + kvh) * hs;
                for (int i = 0; i < hs; i++) acc[i] += p * (double)orc_f16_to_f32(vr[i]);
            }
            for (int i = 0; i < hs; i++) {
                const float o = n > 0 ? (float)(acc[i] / sum) : 0.0f;
                const int64_t at = ((int64_t)s * heads + h) * hs + i;
                if (out) out[at] = orc_f32_to_f16(o);
                if (out_f32) out_f32[at] = o;
            }
        }
        free(logit);
        free(acc);
    }
}
