// Elementwise, row and gather/scatter kernels of a decoder graph (reference:
// crates/kernels/src/cuda/native/core.cu; op semantics are ggml's CPU backend,
// vendor/ggml/src/ggml-cpu/ops.cpp). All of these are HBM-bound: rows are read with 128-bit
// loads where the layout allows it, and the fusions that matter for a decode step (norm*weight,
// act(gate)*up, rope+cast) are single passes.
#include <algorithm>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kernels.h"
#include "dequant.cuh"
#include "pdl.cuh"

namespace tlb {

// ---------------------------------------------------------------- typed element access (reads: dequant.cuh)
__device__ __forceinline__ void st_elem(uint8_t *p, uint32_t ty, float v) {
    switch (ty) {
        case TLB_TYPE_F32: *reinterpret_cast<float *>(p) = v; break;
        case TLB_TYPE_F16: *reinterpret_cast<__half *>(p) = __float2half_rn(v); break;
        case TLB_TYPE_BF16: *reinterpret_cast<__nv_bfloat16 *>(p) = __float2bfloat16_rn(v); break;
        case TLB_TYPE_I32: *reinterpret_cast<int32_t *>(p) = (int32_t)v; break;
        case TLB_TYPE_I64: *reinterpret_cast<int64_t *>(p) = (int64_t)v; break;
        default: break;
    }
}

__device__ __forceinline__ void decomp(int64_t i, const int64_t *ne, int64_t &i0, int64_t &i1, int64_t &i2, int64_t &i3) {
    i0 = i % ne[0]; i /= ne[0];
    i1 = i % ne[1]; i /= ne[1];
    i2 = i % ne[2];
    i3 = i / ne[2];
}
__device__ __forceinline__ int64_t offs(const TView &t, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    return i0 * t.nb[0] + i1 * t.nb[1] + i2 * t.nb[2] + i3 * t.nb[3];
}

__device__ __forceinline__ float block_sum(float v, float *sh) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[w] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < nw; i++) r += sh[i];
    return r;
}
__device__ __forceinline__ float block_max(float v, float *sh) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[w] = v;
    __syncthreads();
    float r = -CUDART_INF_F;
    for (int i = 0; i < nw; i++) r = fmaxf(r, sh[i]);
    return r;
}

static inline unsigned nblocks(int64_t n, int per) { return (unsigned)((n + per - 1) / per > 0 ? (n + per - 1) / per : 1); }
static inline int row_threads(int64_t n) {
    int t = 32;
    while (t < 256 && t < n) t <<= 1;
    return t;
}

// ---------------------------------------------------------------- ADD/SUB/MUL/DIV (f32, ggml broadcast)
__device__ __forceinline__ float bin_op(int op, float a, float b) {
    return op == 0 ? a + b : op == 1 ? a - b : op == 2 ? a * b : a / b;
}
__global__ void k_bin(BinArgs p, const uint8_t *a, const uint8_t *b, uint8_t *d, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        decomp(i, p.d.ne, i0, i1, i2, i3);
        const float x = *reinterpret_cast<const float *>(a + offs(p.a, i0, i1, i2, i3));
        const float y = *reinterpret_cast<const float *>(b + offs(p.b, i0 % p.b.ne[0], i1 % p.b.ne[1], i2 % p.b.ne[2], i3 % p.b.ne[3]));
        *reinterpret_cast<float *>(d + offs(p.d, i0, i1, i2, i3)) = bin_op(p.op, x, y);
    }
}
// contiguous a and d, b either the same shape or one row repeated: 128-bit accesses
__global__ void k_bin_vec(int op, const float4 *a, const float4 *b, float4 *d, int64_t n4, int64_t bn4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 x = a[i], y = b[i % bn4];
        d[i] = make_float4(bin_op(op, x.x, y.x), bin_op(op, x.y, y.y), bin_op(op, x.z, y.z), bin_op(op, x.w, y.w));
    }
}
static bool contiguous_f32(const TView &t) {
    int64_t s = 4;
    for (int i = 0; i < 4; i++) {
        if (t.ne[i] != 1 && t.nb[i] != s) return false;
        s *= t.ne[i];
    }
    return true;
}
cudaError_t launch_bin(const BinArgs &p, const void *a, const void *b, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    const int64_t bn = p.b.ne[0] * p.b.ne[1] * p.b.ne[2] * p.b.ne[3];
    const bool same = p.b.ne[0] == p.d.ne[0] && p.b.ne[1] == p.d.ne[1] && p.b.ne[2] == p.d.ne[2] && p.b.ne[3] == p.d.ne[3];
    const bool row = p.b.ne[0] == p.d.ne[0] && bn == p.b.ne[0];
    if (contiguous_f32(p.a) && contiguous_f32(p.d) && contiguous_f32(p.b) && (same || row) && p.d.ne[0] % 4 == 0 &&
        ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)d % 16 == 0)) {
        k_bin_vec<<<nblocks(n / 4, 256), 256, 0, st>>>(p.op, (const float4 *)a, (const float4 *)b, (float4 *)d, n / 4, bn / 4);
    } else {
        k_bin<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (const uint8_t *)b, (uint8_t *)d, n);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------- UNARY / SCALE / CLAMP / ...
// codes 0..21 are ggml's enum ggml_unary_op; 100.. are the other single-source ops
// (crates/kernels/src/cuda/lower.rs:252-290 uses the same numbering).
__device__ __forceinline__ float unary_op(int code, float x, float p0, float p1) {
    switch (code) {
        case 0: return fabsf(x);
        case 1: return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f);
        case 2: return -x;
        case 3: return x > 0.f ? 1.f : 0.f;
        case 4: return tanhf(x);
        case 5: return x > 0.f ? x : expm1f(x);
        case 6: return x > 0.f ? x : 0.f;
        case 7: return 1.f / (1.f + expf(-x));
        case 8: return 0.5f * x * (1.f + tanhf(0.79788456080286535587989211986876f * x * (1.f + 0.044715f * x * x)));
        case 9: return x * (1.f / (1.f + expf(-1.702f * x)));
        case 10: return x / (1.f + expf(-x));
        case 11: return x * fminf(1.f, fmaxf(0.f, (x + 3.f) / 6.f));
        case 12: return fminf(1.f, fmaxf(0.f, (x + 3.f) / 6.f));
        case 13: return expf(x);
        case 14: return expm1f(x);
        case 15: return x > 20.f ? x : logf(1.f + expf(x));
        case 16: return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
        case 18: return floorf(x);
        case 19: return ceilf(x);
        case 20: return roundf(x);
        case 21: return truncf(x);
        case 100: return x * p0 + p1;
        case 101: return p0;
        case 102: return fminf(fmaxf(x, p0), p1);
        case 103: return x > 0.f ? x : x * p0;
        case 104: return x * x;
        case 105: return sqrtf(x);
        case 106: return sinf(x);
        case 107: return cosf(x);
        case 108: return logf(x);
        default: return x;
    }
}
__global__ void k_unary(UnaryArgs p, const uint8_t *a, uint8_t *d, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        decomp(i, p.d.ne, i0, i1, i2, i3);
        const float x = ld_elem(a + offs(p.a, i0, i1, i2, i3), p.aty);
        st_elem(d + offs(p.d, i0, i1, i2, i3), p.dty, unary_op(p.code, x, p.p0, p.p1));
    }
}
cudaError_t launch_unary(const UnaryArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_unary<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d, n);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- GLU: d = act(a) * b
__device__ __forceinline__ float glu_act(int op, float x) {
    switch (op) {
        case 0: return x > 0.f ? x : 0.f;
        case 1: return unary_op(8, x, 0, 0);
        case 2: return x / (1.f + expf(-x));
        case 4: return unary_op(16, x, 0, 0);
        case 5: return unary_op(9, x, 0, 0);
        default: return x;
    }
}
__global__ void k_glu(GluArgs p, const float *a, const float *b, float *d) {
    const int64_t total = p.n * p.rows;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / p.n, c = i % p.n;
        d[i] = glu_act(p.glu_op, a[r * p.lda + c]) * b[r * p.ldb + c];
    }
}
// Prompt-sized operands (hundreds of MB): four columns per thread, 128-bit accesses
__global__ void k_glu4(GluArgs p, const float *a, const float *b, float *d) {
    const int64_t n4 = p.n / 4, total = n4 * p.rows;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n4, c = (i - r * n4) * 4;
        const float4 x = *reinterpret_cast<const float4 *>(a + r * p.lda + c);
        const float4 y = *reinterpret_cast<const float4 *>(b + r * p.ldb + c);
        float4 o;
        o.x = glu_act(p.glu_op, x.x) * y.x;
        o.y = glu_act(p.glu_op, x.y) * y.y;
        o.z = glu_act(p.glu_op, x.z) * y.z;
        o.w = glu_act(p.glu_op, x.w) * y.w;
        *reinterpret_cast<float4 *>(d + r * p.n + c) = o;
    }
}
cudaError_t launch_glu(const GluArgs &p, const float *a, const float *b, float *d, cudaStream_t st) {
    if (p.n * p.rows == 0) return cudaSuccess;
    const bool vec = p.n % 4 == 0 && p.lda % 4 == 0 && p.ldb % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)d) & 15) == 0;
    if (vec) {
        k_glu4<<<nblocks(p.n / 4 * p.rows, 256), 256, 0, st>>>(p, a, b, d);
        return cudaGetLastError();
    }
    k_glu<<<nblocks(p.n * p.rows, 256), 256, 0, st>>>(p, a, b, d);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- NORM / RMS_NORM (* weight)
// One CTA per row, the row stays in registers between the reduction and the scaling pass
// (up to 16 values per thread; longer rows are re-read from L2).
__global__ void k_norm(NormArgs p, const uint8_t *a, const uint8_t *w, uint8_t *d) {
    __shared__ float sh[32];
    const int64_t row = blockIdx.x;
    const int64_t i1 = row % p.a.ne[1], i2 = (row / p.a.ne[1]) % p.a.ne[2], i3 = row / (p.a.ne[1] * p.a.ne[2]);
    const float *x = reinterpret_cast<const float *>(a + i1 * p.a.nb[1] + i2 * p.a.nb[2] + i3 * p.a.nb[3]);
    float *y = reinterpret_cast<float *>(d + i1 * p.d.nb[1] + i2 * p.d.nb[2] + i3 * p.d.nb[3]);
    const int64_t n = p.a.ne[0];
    const float *wr = nullptr;
    if (p.has_w)
        wr = reinterpret_cast<const float *>(w + (i1 % p.w.ne[1]) * p.w.nb[1] + (i2 % p.w.ne[2]) * p.w.nb[2] + (i3 % p.w.ne[3]) * p.w.nb[3]);
    const int64_t wn = p.has_w ? p.w.ne[0] : 1;
    float v[16];
    const bool cached = n <= (int64_t)blockDim.x * 16;
    float s = 0.f, s1 = 0.f;
    int c = 0;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x, c++) {
        const float t = x[i];
        if (cached) v[c & 15] = t;
        s += t * t;
        s1 += t;
    }
    float mean = 0.f, scale;
    if (p.rms) {
        s = block_sum(s, sh);
        scale = 1.0f / sqrtf(s / (float)n + p.eps);
    } else {
        mean = block_sum(s1, sh) / (float)n;
        float var = 0.f;
        c = 0;
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x, c++) {
            const float t = (cached ? v[c & 15] : x[i]) - mean;
            var += t * t;
        }
        var = block_sum(var, sh) / (float)n;
        scale = 1.0f / sqrtf(var + p.eps);
    }
    c = 0;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x, c++) {
        float t = ((cached ? v[c & 15] : x[i]) - mean) * scale;
        if (wr) t *= wr[wn == n ? i : (int64_t)((uint32_t)i % (uint32_t)wn)];
        y[i] = t;
    }
}
cudaError_t launch_norm(const NormArgs &p, const void *a, const void *w, void *d, cudaStream_t st) {
    const int64_t rows = p.a.ne[1] * p.a.ne[2] * p.a.ne[3];
    if (rows == 0 || p.a.ne[0] == 0) return cudaSuccess;
    k_norm<<<(unsigned)rows, row_threads(p.a.ne[0]), 0, st>>>(p, (const uint8_t *)a, (const uint8_t *)w, (uint8_t *)d);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- ROPE (normal and neox pairs, YaRN ramp)
// theta is built the way the CPU backend builds its cache (ops.cpp:5846-5860): multiplied up
// sequentially in f32, not powf, so long positions agree.
// cos/sin of pair `pr` at position `posf` (rope_yarn, ops.cpp:5806-5830)
__device__ __forceinline__ void rope_cs(const RopeArgs &p, int64_t pr, float posf, const float *ff, float &cs, float &sn) {
    float theta = posf;
    for (int64_t k = 0; k < pr; k++) theta *= p.theta_scale;
    const float fq = p.has_ff ? ff[pr] : 1.0f;
    const float theta_extrap = theta / fq;
    const float theta_interp = p.freq_scale * theta_extrap;
    float th = theta_interp, mscale = p.attn_factor;
    if (p.ext_factor != 0.0f) {
        const float yv = ((float)pr - p.corr0) / fmaxf(0.001f, p.corr1 - p.corr0);
        const float ramp_mix = (1.f - fminf(1.f, fmaxf(0.f, yv))) * p.ext_factor;
        // two rounded products and a rounded sum, as the CPU build computes it: at position 4096 one unit in the last
        // place of the angle is 5e-4 rad, so a fused multiply-add here shows in the fourth digit of the result
        th = __fadd_rn(__fmul_rn(theta_interp, 1.f - ramp_mix), __fmul_rn(theta_extrap, ramp_mix));
        mscale *= 1.0f + 0.1f * logf(1.0f / p.freq_scale);
    }
    cs = cosf(th) * mscale;
    sn = sinf(th) * mscale;
}

// A thread owns one (pair, position) and walks `hc` heads with it: cos and sin depend on the position and the pair
// only, and the sequential product behind theta is the costly part (a prompt of 16k tokens has 32 heads per position).
__global__ void k_rope(RopeArgs p, const uint8_t *a, const int32_t *pos, const float *ff, uint8_t *d, int64_t npairs, int hc) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    const int64_t half = p.a.ne[0] / 2;
    const int64_t pr = i % half;
    int64_t r = i / half;
    const int64_t i2 = r % p.a.ne[2];
    const int64_t i3 = r / p.a.ne[2];
    const int64_t h0 = (int64_t)blockIdx.y * hc, h1 = min(h0 + hc, p.a.ne[1]);
    const uint8_t *src = a + i2 * p.a.nb[2] + i3 * p.a.nb[3];
    uint8_t *dst = d + i2 * p.d.nb[2] + i3 * p.d.nb[3];
    const int64_t i0 = 2 * pr;
    if (i0 >= p.n_dims) {  // dims past n_dims are copied through
        for (int64_t i1 = h0; i1 < h1; i1++) {
            st_elem(dst + i1 * p.d.nb[1] + i0 * p.d.nb[0], p.dty, ld_elem(src + i1 * p.a.nb[1] + i0 * p.a.nb[0], p.aty));
            st_elem(dst + i1 * p.d.nb[1] + (i0 + 1) * p.d.nb[0], p.dty, ld_elem(src + i1 * p.a.nb[1] + (i0 + 1) * p.a.nb[0], p.aty));
        }
        return;
    }
    float cs, sn;
    rope_cs(p, pr, (float)pos[i2], ff, cs, sn);
    const int64_t ic = p.mode == 0 ? i0 : pr;
    const int64_t off = p.mode == 0 ? 1 : p.n_dims / 2;
    for (int64_t i1 = h0; i1 < h1; i1++) {
        const uint8_t *s1 = src + i1 * p.a.nb[1];
        uint8_t *d1 = dst + i1 * p.d.nb[1];
        const float x0 = ld_elem(s1 + ic * p.a.nb[0], p.aty), x1 = ld_elem(s1 + (ic + off) * p.a.nb[0], p.aty);
        st_elem(d1 + ic * p.d.nb[0], p.dty, x0 * cs - x1 * sn);
        st_elem(d1 + (ic + off) * p.d.nb[0], p.dty, x0 * sn + x1 * cs);
    }
}

// One launch for the attention inputs of a decode step: rope(q) -> f16 query, rope(k) -> f16 into
// the key pool at the token's slot, v -> f16 into the value pool. Same arithmetic as k_rope followed
// by the f32 -> f16 casts and the cache write; a negative slot skips the token's key and value.
__global__ void k_rope_kv(RopeKvArgs p, const uint8_t *q, const uint8_t *k, const uint8_t *v, const int32_t *pos,
                          const float *ff, __half *q16, __half *kpool, __half *vpool, const int64_t *slots, int *err) {
    griddep_launch();
    griddep_wait();
    const int tok = blockIdx.x, hsl = blockIdx.y, pr = threadIdx.x;
    const int hs = p.hs;
    if (hsl < p.heads + p.kv_heads) {
        const bool is_q = hsl < p.heads;
        const int h = is_q ? hsl : hsl - p.heads;
        const uint8_t *src;
        __half *dst;
        if (is_q) {
            src = q + h * p.rope.a.nb[1] + tok * p.rope.a.nb[2];
            dst = q16 + ((size_t)tok * p.heads + h) * hs;
        } else {
            const int64_t slot = slots[tok];
            if (slot < 0) return;
            if (slot >= p.pool_slots) {   // beyond the pools: nothing is written, the host hears of it
                if (pr == 0 && err) atomicExch(err, TLB_ERR_INDEX);
                return;
            }
            src = k + h * p.k.nb[1] + tok * p.k.nb[2];
            dst = kpool + (((size_t)(slot / p.block_size) * p.kv_heads + h) * p.block_size + slot % p.block_size) * hs;
        }
        const float *x = reinterpret_cast<const float *>(src);
        const int i0 = 2 * pr;
        if (i0 >= p.rope.n_dims) {
            dst[i0] = __float2half_rn(x[i0]);
            dst[i0 + 1] = __float2half_rn(x[i0 + 1]);
            return;
        }
        float cs, sn;
        rope_cs(p.rope, pr, (float)pos[tok], ff, cs, sn);
        const int ic = p.rope.mode == 0 ? i0 : pr;
        const int off = p.rope.mode == 0 ? 1 : p.rope.n_dims / 2;
        const float x0 = x[ic], x1 = x[ic + off];
        dst[ic] = __float2half_rn(x0 * cs - x1 * sn);
        dst[ic + off] = __float2half_rn(x0 * sn + x1 * cs);
    } else {
        const int64_t slot = slots[tok];
        if (slot < 0 || slot >= p.pool_slots) return;   // reported by the key's CTA
        const int h = hsl - p.heads - p.kv_heads;
        const float2 x = *reinterpret_cast<const float2 *>(v + h * p.v.nb[1] + tok * p.v.nb[2] + pr * 8);
        __half *dst = vpool + (((size_t)(slot / p.block_size) * p.kv_heads + h) * p.block_size + slot % p.block_size) * hs;
        *reinterpret_cast<__half2 *>(dst + 2 * pr) = __floats2half2_rn(x.x, x.y);
    }
}
cudaError_t launch_rope_kv(const RopeKvArgs &p, const void *q, const void *k, const void *v, const int32_t *pos, const float *ff,
                           void *q16, void *kpool, void *vpool, const int64_t *slots, int *err, cudaStream_t st) {
    if (p.tokens == 0) return cudaSuccess;
    return launch_pdl(k_rope_kv, dim3((unsigned)p.tokens, (unsigned)(p.heads + 2 * p.kv_heads)), dim3(p.hs / 2), 0, st, p,
                      (const uint8_t *)q, (const uint8_t *)k, (const uint8_t *)v, pos, ff, (__half *)q16, (__half *)kpool, (__half *)vpool, slots, err);
}
cudaError_t launch_rope(const RopeArgs &p, const void *a, const int32_t *pos, const float *ff, void *d, cudaStream_t st) {
    const int64_t n = p.a.ne[0] / 2 * p.a.ne[2] * p.a.ne[3];   // (pair, position) units
    if (n == 0 || p.a.ne[1] == 0) return cudaSuccess;
    // heads per thread: all of them once the units alone fill the GPU, one each for short inputs
    int hc = (int)std::max<int64_t>(1, std::min<int64_t>(p.a.ne[1], n / 65536));
    hc = (int)std::max<int64_t>(hc, (p.a.ne[1] + 65534) / 65535);   // grid.y stays below its limit
    const dim3 grid(nblocks(n, 256), (unsigned)((p.a.ne[1] + hc - 1) / hc));
    k_rope<<<grid, 256, 0, st>>>(p, (const uint8_t *)a, pos, ff, (uint8_t *)d, n, hc);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- SOFT_MAX (scale, mask, ALiBi)
__global__ void k_soft_max(SoftmaxArgs p, const uint8_t *a, const uint8_t *m, uint8_t *d) {
    __shared__ float sh[32];
    const int64_t row = blockIdx.x;
    const int64_t i1 = row % p.a.ne[1], i2 = (row / p.a.ne[1]) % p.a.ne[2], i3 = row / (p.a.ne[1] * p.a.ne[2]);
    const float *x = reinterpret_cast<const float *>(a + i1 * p.a.nb[1] + i2 * p.a.nb[2] + i3 * p.a.nb[3]);
    float *y = reinterpret_cast<float *>(d + i1 * p.d.nb[1] + i2 * p.d.nb[2] + i3 * p.d.nb[3]);
    const int64_t n = p.a.ne[0];
    const uint8_t *mr = nullptr;
    if (p.has_mask) mr = m + i1 * p.m.nb[1] + (i2 % p.m.ne[2]) * p.m.nb[2] + (i3 % p.m.ne[3]) * p.m.nb[3];
    float slope = 1.0f;
    if (p.max_bias > 0.0f) {
        const int h = (int)i2;
        slope = h < p.n_head_log2 ? powf(p.m0, (float)(h + 1)) : powf(p.m1, (float)(2 * (h - p.n_head_log2) + 1));
    }
    float mx = -CUDART_INF_F;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i] * p.scale;
        if (mr) v += slope * ld_elem(mr + i * p.m.nb[0], p.mty);
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, sh);
    float sum = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i] * p.scale;
        if (mr) v += slope * ld_elem(mr + i * p.m.nb[0], p.mty);
        const float e = expf(v - mx);
        y[i] = e;
        sum += e;
    }
    sum = block_sum(sum, sh);
    const float inv = 1.0f / sum;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) y[i] *= inv;
}
cudaError_t launch_soft_max(const SoftmaxArgs &p, const void *a, const void *m, void *d, cudaStream_t st) {
    const int64_t rows = p.a.ne[1] * p.a.ne[2] * p.a.ne[3];
    if (rows == 0 || p.a.ne[0] == 0) return cudaSuccess;
    k_soft_max<<<(unsigned)rows, row_threads(p.a.ne[0]), 0, st>>>(p, (const uint8_t *)a, (const uint8_t *)m, (uint8_t *)d);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- GET_ROWS / SET_ROWS
__device__ __forceinline__ int64_t ld_index(const uint8_t *p, uint32_t ty) {
    return ty == TLB_TYPE_I64 ? *reinterpret_cast<const int64_t *>(p) : (int64_t)*reinterpret_cast<const int32_t *>(p);
}
// d[:, i10, i11, i12] = a[:, ids[i10, i11, i12], i11, i12]
__global__ void k_get_rows(RowsArgs p, const uint8_t *a, const uint8_t *ids, uint8_t *d) {
    const int64_t r = blockIdx.x;
    const int64_t i10 = r % p.ids.ne[0], i11 = (r / p.ids.ne[0]) % p.ids.ne[1], i12 = r / (p.ids.ne[0] * p.ids.ne[1]);
    const int64_t row = ld_index(ids + i10 * p.ids.nb[0] + i11 * p.ids.nb[1] + i12 * p.ids.nb[2], p.idty);
    const uint8_t *src = a + row * p.a.nb[1] + i11 * p.a.nb[2] + i12 * p.a.nb[3];
    uint8_t *dst = d + i10 * p.d.nb[1] + i11 * p.d.nb[2] + i12 * p.d.nb[3];
    const bool q = is_quant(p.aty);
    for (int64_t i = threadIdx.x; i < p.d.ne[0]; i += blockDim.x) {
        const float v = q ? dq_elem(src, p.aty, i) : ld_elem(src + i * p.a.nb[0], p.aty);
        st_elem(dst + i * p.d.nb[0], p.dty, v);
    }
}
cudaError_t launch_get_rows(const RowsArgs &p, const void *a, const void *ids, void *d, cudaStream_t st) {
    const int64_t rows = p.ids.ne[0] * p.ids.ne[1] * p.ids.ne[2];
    if (rows == 0 || p.d.ne[0] == 0) return cudaSuccess;
    k_get_rows<<<(unsigned)rows, 256, 0, st>>>(p, (const uint8_t *)a, (const uint8_t *)ids, (uint8_t *)d);
    return cudaGetLastError();
}
// d[:, ids[i1, i2 % ne11, i3 % ne12], i2, i3] = rows[:, i1, i2, i3]   (ggml_set_rows)
__global__ void k_set_rows(RowsArgs p, const uint8_t *a, const uint8_t *ids, uint8_t *d) {
    const int64_t r = blockIdx.x;
    const int64_t i1 = r % p.a.ne[1], i2 = (r / p.a.ne[1]) % p.a.ne[2], i3 = r / (p.a.ne[1] * p.a.ne[2]);
    const int64_t row = ld_index(ids + i1 * p.ids.nb[0] + (i2 % p.ids.ne[1]) * p.ids.nb[1] + (i3 % p.ids.ne[2]) * p.ids.nb[2], p.idty);
    if (row < 0 || row >= p.d.ne[1]) return;
    const uint8_t *src = a + i1 * p.a.nb[1] + i2 * p.a.nb[2] + i3 * p.a.nb[3];
    uint8_t *dst = d + row * p.d.nb[1] + i2 * p.d.nb[2] + i3 * p.d.nb[3];
    for (int64_t i = threadIdx.x; i < p.a.ne[0]; i += blockDim.x)
        st_elem(dst + i * p.d.nb[0], p.dty, ld_elem(src + i * p.a.nb[0], p.aty));
}
cudaError_t launch_set_rows(const RowsArgs &p, const void *rows, const void *ids, void *d, cudaStream_t st) {
    const int64_t n = p.a.ne[1] * p.a.ne[2] * p.a.ne[3];
    if (n == 0 || p.a.ne[0] == 0) return cudaSuccess;
    k_set_rows<<<(unsigned)n, 256, 0, st>>>(p, (const uint8_t *)rows, (const uint8_t *)ids, (uint8_t *)d);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- DUP / CPY / CONT (casts, dequantizing reads)
// Element i of the source (in its own index order) goes to element i of the destination.
__global__ void k_cpy(CpyArgs p, const uint8_t *a, uint8_t *d, int64_t n) {
    const bool q = is_quant(p.aty);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t a0, a1, a2, a3, d0, d1, d2, d3;
        decomp(i, p.a.ne, a0, a1, a2, a3);
        decomp(i, p.d.ne, d0, d1, d2, d3);
        float v;
        if (q) v = dq_elem(a + a1 * p.a.nb[1] + a2 * p.a.nb[2] + a3 * p.a.nb[3], p.aty, a0);
        else v = ld_elem(a + offs(p.a, a0, a1, a2, a3), p.aty);
        st_elem(d + offs(p.d, d0, d1, d2, d3), p.dty, v);
    }
}
// same-type contiguous copy and f32 -> f16 contiguous cast: 128-bit reads
__global__ void k_cpy_f32_f16(const float4 *a, uint2 *d, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 v = a[i];
        const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
        d[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
}
static bool contiguous_ty(const TView &t, int64_t es) {
    int64_t s = es;
    for (int i = 0; i < 4; i++) {
        if (t.ne[i] != 1 && t.nb[i] != s) return false;
        s *= t.ne[i];
    }
    return true;
}
cudaError_t launch_cpy(const CpyArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t n = p.a.ne[0] * p.a.ne[1] * p.a.ne[2] * p.a.ne[3];
    if (n == 0) return cudaSuccess;
    if (p.aty == TLB_TYPE_F32 && p.dty == TLB_TYPE_F16 && contiguous_ty(p.a, 4) && contiguous_ty(p.d, 2) && n % 4 == 0 &&
        (uintptr_t)a % 16 == 0 && (uintptr_t)d % 8 == 0) {
        k_cpy_f32_f16<<<nblocks(n / 4, 256), 256, 0, st>>>((const float4 *)a, (uint2 *)d, n / 4);
        return cudaGetLastError();
    }
    if (p.aty == p.dty && !(p.aty == TLB_TYPE_Q8_0 || p.aty == TLB_TYPE_Q4_0 || p.aty == TLB_TYPE_Q4_K)) {
        const int64_t es = p.aty == TLB_TYPE_F32 || p.aty == TLB_TYPE_I32 ? 4 : (p.aty == TLB_TYPE_I64 ? 8 : 2);
        if (contiguous_ty(p.a, es) && contiguous_ty(p.d, es))
            return cudaMemcpyAsync(d, a, (size_t)(n * es), cudaMemcpyDeviceToDevice, st);
    }
    k_cpy<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d, n);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- ARGMAX (last index among ties, as the CPU)
__global__ void k_argmax(TView a, const uint8_t *x, int32_t *out) {
    __shared__ float smax[32];
    __shared__ int sidx[32];
    const int64_t row = blockIdx.x;
    const float *xr = reinterpret_cast<const float *>(x + row * a.nb[1]);
    float mx = -CUDART_INF_F;
    int idx = 0;
    // a row of logits is half a megabyte read by one CTA: 16-byte loads, several in flight per thread (a thread still
    // meets its elements in rising index order, so ">=" keeps the last of equal maxima)
    const int64_t n4 = ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) ? a.ne[0] / 4 : 0;
    const float4 *x4 = reinterpret_cast<const float4 *>(xr);
    int64_t i4 = threadIdx.x;
    for (; i4 + 3 * (int64_t)blockDim.x < n4; i4 += 4 * (int64_t)blockDim.x) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = x4[i4 + u * (int64_t)blockDim.x];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int base = (int)(4 * (i4 + u * (int64_t)blockDim.x));
            if (v[u].x >= mx) { mx = v[u].x; idx = base; }
            if (v[u].y >= mx) { mx = v[u].y; idx = base + 1; }
            if (v[u].z >= mx) { mx = v[u].z; idx = base + 2; }
            if (v[u].w >= mx) { mx = v[u].w; idx = base + 3; }
        }
    }
    for (; i4 < n4; i4 += blockDim.x) {
        const float4 v = x4[i4];
        const int base = (int)(4 * i4);
        if (v.x >= mx) { mx = v.x; idx = base; }
        if (v.y >= mx) { mx = v.y; idx = base + 1; }
        if (v.z >= mx) { mx = v.z; idx = base + 2; }
        if (v.w >= mx) { mx = v.w; idx = base + 3; }
    }
    for (int64_t i = 4 * n4 + threadIdx.x; i < a.ne[0]; i += blockDim.x) {   // the tail, or everything of an unaligned row
        const float v = xr[i];
        if (v >= mx) { mx = v; idx = (int)i; }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, s);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, s);
        if (om > mx || (om == mx && oi > idx)) { mx = om; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { smax[threadIdx.x >> 5] = mx; sidx[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (smax[w] > mx || (smax[w] == mx && sidx[w] > idx)) { mx = smax[w]; idx = sidx[w]; }
        out[row] = idx;
    }
}
cudaError_t launch_argmax(const TView &a, const void *x, int32_t *out, cudaStream_t st) {
    const int64_t rows = a.ne[1] * a.ne[2] * a.ne[3];
    if (rows == 0) return cudaSuccess;
    k_argmax<<<(unsigned)rows, a.ne[0] >= 16384 ? 1024 : 256, 0, st>>>(a, (const uint8_t *)x, out);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- CONCAT / REPEAT / SUM_ROWS / ARANGE (f32)
__global__ void k_concat(SimpleArgs p, const uint8_t *a, const uint8_t *b, uint8_t *d, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t ix[4];
        decomp(i, p.d.ne, ix[0], ix[1], ix[2], ix[3]);
        const int dim = (int)p.i0;
        float v;
        if (ix[dim] < p.a.ne[dim]) {
            v = *reinterpret_cast<const float *>(a + offs(p.a, ix[0], ix[1], ix[2], ix[3]));
        } else {
            int64_t jx[4] = {ix[0], ix[1], ix[2], ix[3]};
            jx[dim] -= p.a.ne[dim];
            v = *reinterpret_cast<const float *>(b + offs(p.b, jx[0], jx[1], jx[2], jx[3]));
        }
        *reinterpret_cast<float *>(d + offs(p.d, ix[0], ix[1], ix[2], ix[3])) = v;
    }
}
cudaError_t launch_concat(const SimpleArgs &p, const void *a, const void *b, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_concat<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (const uint8_t *)b, (uint8_t *)d, n);
    return cudaGetLastError();
}
__global__ void k_repeat(SimpleArgs p, const uint8_t *a, uint8_t *d, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t i0, i1, i2, i3;
        decomp(i, p.d.ne, i0, i1, i2, i3);
        *reinterpret_cast<float *>(d + offs(p.d, i0, i1, i2, i3)) =
            *reinterpret_cast<const float *>(a + offs(p.a, i0 % p.a.ne[0], i1 % p.a.ne[1], i2 % p.a.ne[2], i3 % p.a.ne[3]));
    }
}
cudaError_t launch_repeat(const SimpleArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_repeat<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d, n);
    return cudaGetLastError();
}
__global__ void k_sum_rows(SimpleArgs p, const uint8_t *a, uint8_t *d) {
    __shared__ float sh[32];
    const int64_t row = blockIdx.x;
    const int64_t i1 = row % p.a.ne[1], i2 = (row / p.a.ne[1]) % p.a.ne[2], i3 = row / (p.a.ne[1] * p.a.ne[2]);
    const float *x = reinterpret_cast<const float *>(a + i1 * p.a.nb[1] + i2 * p.a.nb[2] + i3 * p.a.nb[3]);
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < p.a.ne[0]; i += blockDim.x) s += x[i];
    s = block_sum(s, sh);
    if (threadIdx.x == 0)
        *reinterpret_cast<float *>(d + i1 * p.d.nb[1] + i2 * p.d.nb[2] + i3 * p.d.nb[3]) = p.i0 ? s / (float)p.a.ne[0] : s;
}
cudaError_t launch_sum_rows(const SimpleArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t rows = p.a.ne[1] * p.a.ne[2] * p.a.ne[3];
    if (rows == 0) return cudaSuccess;
    k_sum_rows<<<(unsigned)rows, row_threads(p.a.ne[0]), 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d);
    return cudaGetLastError();
}
__global__ void k_arange(float start, float step, float *d, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = start + step * (float)i;
}
cudaError_t launch_arange(const SimpleArgs &p, void *d, cudaStream_t st) {
    if (p.d.ne[0] == 0) return cudaSuccess;
    k_arange<<<nblocks(p.d.ne[0], 256), 256, 0, st>>>(p.f0, p.f1, (float *)d, p.d.ne[0]);
    return cudaGetLastError();
}

// ---------------------------------------------------------------- image ops
// The reference's native executor runs these one thread per destination element (crates/kernels/src/cuda/native/
// core.cu:240-261 im2col, 285-358 upscale, 405-427 pool_2d, 483-536 conv_2d_dw / pad / pad_reflect_1d); the arithmetic is
// that of ggml's CPU operators (vendor/ggml/src/ggml-cpu/ops.cpp).

// IM2COL: d[n][oh][ow][ic*KH*KW + ky*KW + kx] = x[n][ic][oh*s1 + ky*d1 - p1][ow*s0 + kx*d0 - p0], zero outside
// (1-D: d[n][ow][ic*KW + kx] = x[n][ic][ow*s0 + kx*d0 - p0])
__global__ void k_im2col(Im2colArgs p, const uint8_t *x, uint8_t *d, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t i0, i1, i2, i3;
    decomp(i, p.d.ne, i0, i1, i2, i3);
    const int64_t ow = i1, oh = p.is2d ? i2 : 0, img = p.is2d ? i3 : i2;
    const int64_t khw = p.KW * p.KH, ic = i0 / khw, r = i0 % khw, ky = r / p.KW, kx = r % p.KW;
    const int64_t iy = oh * p.s1 + ky * p.d1 - p.p1, ix = ow * p.s0 + kx * p.d0 - p.p0;
    float v = 0.f;
    if (iy >= 0 && iy < p.IH && ix >= 0 && ix < p.IW)
        v = ld_elem(x + (p.is2d ? img * p.x.nb[3] + ic * p.x.nb[2] + iy * p.x.nb[1] : img * p.x.nb[2] + ic * p.x.nb[1]) + ix * p.x.nb[0], p.xty);
    st_elem(d + offs(p.d, i0, i1, i2, i3), p.dty, v);
}
cudaError_t launch_im2col(const Im2colArgs &p, const void *x, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_im2col<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)x, (uint8_t *)d, n);
    return cudaGetLastError();
}

// UPSCALE (ggml_compute_forward_upscale_f32, ops.cpp:7832-8024): nearest, bilinear (optionally antialiased), bicubic
__device__ __forceinline__ float cubic_w1(float x) { return ((-0.75f + 2.f) * x - (-0.75f + 3.f)) * x * x + 1.f; }
__device__ __forceinline__ float cubic_w2(float x) { return ((-0.75f * x - 5.f * -0.75f) * x + 8.f * -0.75f) * x - 4.f * -0.75f; }
__device__ __forceinline__ float cubic4(float p0, float p1, float p2, float p3, float x) {
    return p0 * cubic_w2(x + 1.f) + p1 * cubic_w1(x) + p2 * cubic_w1(1.f - x) + p3 * cubic_w2(2.f - x);
}
__global__ void k_upscale(UpscaleArgs p, const uint8_t *a, uint8_t *d, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t i0, i1, i2, i3;
    decomp(i, p.d.ne, i0, i1, i2, i3);
    const int64_t w = p.a.ne[0], h = p.a.ne[1];
    const uint8_t *plane = a + (int64_t)((float)i2 / p.sf2) * p.a.nb[2] + (int64_t)((float)i3 / p.sf3) * p.a.nb[3];
    auto px = [&](int64_t xx, int64_t yy) { return *reinterpret_cast<const float *>(plane + xx * p.a.nb[0] + yy * p.a.nb[1]); };
    auto clampi = [](int64_t v, int64_t hi) { return v < 0 ? (int64_t)0 : (v > hi ? hi : v); };
    float val;
    if (p.mode == 0) {
        val = px((int64_t)((float)i0 / p.sf0), (int64_t)((float)i1 / p.sf1));
    } else if (p.mode == 1 && p.antialias) {
        const float sup1 = fmaxf(1.0f, 1.0f / p.sf1), inv1 = 1.0f / sup1, sup0 = fmaxf(1.0f, 1.0f / p.sf0), inv0 = 1.0f / sup0;
        const float y = ((float)i1 + p.poff) / p.sf1, x = ((float)i0 + p.poff) / p.sf0;
        const int64_t x_min = max((int64_t)(x - sup0 + p.poff), (int64_t)0), x_max = min((int64_t)(x + sup0 + p.poff), w);
        const int64_t y_min = max((int64_t)(y - sup1 + p.poff), (int64_t)0), y_max = min((int64_t)(y + sup1 + p.poff), h);
        float sum = 0.f, total = 0.f;
        for (int64_t sy = y_min; sy < y_max; sy++) {
            const float wy = fmaxf(1.0f - fabsf(((float)sy - y + p.poff) * inv1), 0.0f);
            for (int64_t sx = x_min; sx < x_max; sx++) {
                const float wx = fmaxf(1.0f - fabsf(((float)sx - x + p.poff) * inv0), 0.0f);
                const float wt = wx * wy;
                if (wt <= 0.0f) continue;
                sum += px(sx, sy) * wt;
                total += wt;
            }
        }
        val = total > 0.f ? sum / total : sum;
    } else if (p.mode == 1) {
        const float y = ((float)i1 + p.poff) / p.sf1 - p.poff, x = ((float)i0 + p.poff) / p.sf0 - p.poff;
        const int64_t yf = (int64_t)floorf(y), xf = (int64_t)floorf(x);
        const int64_t y0 = clampi(yf, h - 1), y1 = clampi(yf + 1, h - 1), x0 = clampi(xf, w - 1), x1 = clampi(xf + 1, w - 1);
        const float dy = fmaxf(0.0f, fminf(y - (float)y0, 1.0f)), dx = fmaxf(0.0f, fminf(x - (float)x0, 1.0f));
        val = px(x0, y0) * (1 - dx) * (1 - dy) + px(x1, y0) * dx * (1 - dy) + px(x0, y1) * (1 - dx) * dy + px(x1, y1) * dx * dy;
    } else {
        const float y = ((float)i1 + p.poff) / p.sf1 - p.poff, x = ((float)i0 + p.poff) / p.sf0 - p.poff;
        const int64_t y0 = (int64_t)floorf(y), x0 = (int64_t)floorf(x);
        const float dy = y - (float)y0, dx = x - (float)x0;
        float rows[4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int64_t yy = clampi(y0 + r - 1, h - 1);
            rows[r] = cubic4(px(clampi(x0 - 1, w - 1), yy), px(clampi(x0, w - 1), yy), px(clampi(x0 + 1, w - 1), yy), px(clampi(x0 + 2, w - 1), yy), dx);
        }
        val = cubic4(rows[0], rows[1], rows[2], rows[3], dy);
    }
    *reinterpret_cast<float *>(d + offs(p.d, i0, i1, i2, i3)) = val;
}
cudaError_t launch_upscale(const UpscaleArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_upscale<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d, n);
    return cudaGetLastError();
}

// POOL_2D: max (kind 0) or average over the k0 x k1 window (kind 1; the divisor is the whole window, as on the CPU)
__global__ void k_pool_2d(Pool2dArgs p, const uint8_t *a, uint8_t *d, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t i0, i1, i2, i3;
    decomp(i, p.d.ne, i0, i1, i2, i3);
    const uint8_t *plane = a + i2 * p.a.nb[2] + i3 * p.a.nb[3];
    const int64_t ix = i0 * p.s0 - p.p0, iy = i1 * p.s1 - p.p1;
    float res = p.kind == 1 ? 0.f : -3.402823466e+38f;
    for (int ky = 0; ky < p.k1; ky++) {
        if (iy + ky < 0 || iy + ky >= p.a.ne[1]) continue;
        for (int kx = 0; kx < p.k0; kx++) {
            if (ix + kx < 0 || ix + kx >= p.a.ne[0]) continue;
            const float v = ld_elem(plane + (iy + ky) * p.a.nb[1] + (ix + kx) * p.a.nb[0], p.aty);
            res = p.kind == 1 ? res + v : fmaxf(v, res);
        }
    }
    if (p.kind == 1) res /= (float)(p.k0 * p.k1);
    st_elem(d + offs(p.d, i0, i1, i2, i3), p.dty, res);
}
cudaError_t launch_pool_2d(const Pool2dArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_pool_2d<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d, n);
    return cudaGetLastError();
}

// CONV_2D_DW: depthwise convolution, kernel [KW, KH, 1, C] over data [W, H, C, N]
__global__ void k_conv_2d_dw(ConvDwArgs p, const uint8_t *k, const uint8_t *x, uint8_t *d, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t i0, i1, i2, i3;
    decomp(i, p.d.ne, i0, i1, i2, i3);
    const uint8_t *xp = x + i2 * p.x.nb[2] + i3 * p.x.nb[3], *kp = k + i2 * p.k.nb[3];
    float sum = 0.f;
    for (int64_t ky = 0; ky < p.k.ne[1]; ky++) {
        const int64_t iy = i1 * p.s1 + ky * p.d1 - p.p1;
        if (iy < 0 || iy >= p.x.ne[1]) continue;
        for (int64_t kx = 0; kx < p.k.ne[0]; kx++) {
            const int64_t ix = i0 * p.s0 + kx * p.d0 - p.p0;
            if (ix < 0 || ix >= p.x.ne[0]) continue;
            sum += ld_elem(xp + iy * p.x.nb[1] + ix * p.x.nb[0], p.xty) * ld_elem(kp + ky * p.k.nb[1] + kx * p.k.nb[0], p.kty);
        }
    }
    st_elem(d + offs(p.d, i0, i1, i2, i3), p.dty, sum);
}
cudaError_t launch_conv_2d_dw(const ConvDwArgs &p, const void *k, const void *x, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_conv_2d_dw<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)k, (const uint8_t *)x, (uint8_t *)d, n);
    return cudaGetLastError();
}

// PAD (zeros around the source, lp[] elements in front of each dimension) and PAD_REFLECT_1D (dimension 0 mirrored);
// elements are copied as bytes (2 or 4), so every plain type passes through unchanged
__global__ void k_pad(PadArgs p, const uint8_t *a, uint8_t *d, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t i0, i1, i2, i3;
    decomp(i, p.d.ne, i0, i1, i2, i3);
    int64_t j0 = i0 - p.lp[0], j1 = i1 - p.lp[1], j2 = i2 - p.lp[2], j3 = i3 - p.lp[3];
    bool inside = true;
    if (p.reflect) {
        if (j0 < 0) j0 = -j0;
        if (j0 >= p.a.ne[0]) j0 = 2 * (p.a.ne[0] - 1) - j0;
    } else {
        inside = j0 >= 0 && j0 < p.a.ne[0] && j1 >= 0 && j1 < p.a.ne[1] && j2 >= 0 && j2 < p.a.ne[2] && j3 >= 0 && j3 < p.a.ne[3];
    }
    uint8_t *dp = d + offs(p.d, i0, i1, i2, i3);
    const uint8_t *sp = a + (inside ? offs(p.a, j0, j1, j2, j3) : 0);
    if (p.elem_bytes == 4) *reinterpret_cast<uint32_t *>(dp) = inside ? *reinterpret_cast<const uint32_t *>(sp) : 0u;
    else *reinterpret_cast<uint16_t *>(dp) = inside ? *reinterpret_cast<const uint16_t *>(sp) : (uint16_t)0;
}
cudaError_t launch_pad(const PadArgs &p, const void *a, void *d, cudaStream_t st) {
    const int64_t n = p.d.ne[0] * p.d.ne[1] * p.d.ne[2] * p.d.ne[3];
    if (n == 0) return cudaSuccess;
    k_pad<<<nblocks(n, 256), 256, 0, st>>>(p, (const uint8_t *)a, (uint8_t *)d, n);
    return cudaGetLastError();
}

}  // namespace tlb
