// FLASH_ATTN_EXT: dense attention softmax(scale * Q K^T + slope * mask) V for prefill and for caches that
// are ordinary tensors (reference: crates/kernels/src/cuda/lower.rs:575-657 and native/fa.cu; semantics of
// ggml_compute_forward_flash_attn_ext_f16, vendor/ggml/src/ggml-cpu/ops.cpp).
//
//   q f32 [D, nq, nh, nb]   k [D, nkv, nhkv, nb]   v [Dv, nkv, nhkv, nb] (f16 or f32)
//   mask f16 [nkv, >= nq, ne32, ne33] or none      out f32 [Dv, nh, nq, nb]
//
// A CTA of four warps owns 64 consecutive queries of one (head, batch); each warp keeps 16 of them as
// the M rows of mma.sync.m16n8k16 (f16 operands, f32 accumulate): the queries live in registers as A
// fragments for the whole kernel, 64-key tiles of K and V are staged in shared memory as f16 (rows
// padded by 16 bytes, so fragment loads and ldmatrix are conflict-free), S = Q K^T, online softmax in
// base 2 on the accumulator fragments, P goes back in as the A operand of O += P V. Like the CPU
// backend with an f16 cache, q is rounded to f16 before the dot products.
#include <algorithm>
#include <cstdlib>
#include <string>

#include <cuda_fp16.h>
#include <math_constants.h>

#include "dequant.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace tlb {

namespace {

constexpr int FA_WARPS = 4;
constexpr int FA_QT = 16 * FA_WARPS;   // queries per CTA
constexpr int FA_KT = 64;              // keys per tile

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t &r0, uint32_t &r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// one row of K or V (D elements, f16 or f32 in global memory) -> f16 in shared memory, 8 elements per call
template <bool F32>
__device__ __forceinline__ void stage8(__half *dst, const uint8_t *src, bool live) {
    uint4 out = make_uint4(0, 0, 0, 0);
    if (live) {
        if (F32) {
            const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 16);
            out = make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(b.x, b.y), pack_h2(b.z, b.w));
        } else {
            out = *reinterpret_cast<const uint4 *>(src);
        }
    }
    *reinterpret_cast<uint4 *>(dst) = out;
}

template <int D, bool KF32, bool VF32>
__global__ void __launch_bounds__(FA_WARPS * 32) k_flash_attn(FlashArgs p, const uint8_t *__restrict__ q, const uint8_t *__restrict__ k,
                                                              const uint8_t *__restrict__ v, const uint8_t *__restrict__ mask,
                                                              float *__restrict__ out, float *__restrict__ partial) {
    griddep_launch();
    griddep_wait();
    constexpr int LDS = D + 8;                 // padded row length in halves
    constexpr int KS = D / 16;                 // k-steps of Q K^T
    constexpr int ND = D / 8;                  // n-tiles of P V
    __shared__ __align__(16) __half Ks[FA_KT * LDS];
    __shared__ __align__(16) __half Vs[FA_KT * LDS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = blockIdx.x % p.parts;           // stretch of the keys this CTA covers (all of them without a split)
    const int q0 = (blockIdx.x / p.parts) * FA_QT + warp * 16;   // first query of this warp
    const int k_begin = part * p.part_len, k_end = min(p.nkv, k_begin + p.part_len);
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.nh / p.nhkv);
    const int qr0 = q0 + (lane >> 2), qr1 = qr0 + 8;  // the two query rows this lane holds pieces of
    const int cq = (lane & 3) * 2;                    // column pair inside an 8-wide tile

    // ---- queries -> A fragments (rounded to f16), kept for the whole kernel
    uint32_t qa[KS][4];
    {
        const uint8_t *qb = q + (int64_t)h * p.q.nb[2] + (int64_t)b * p.q.nb[3];
        const float *r0 = reinterpret_cast<const float *>(qb + (int64_t)min(qr0, p.nq - 1) * p.q.nb[1]);
        const float *r1 = reinterpret_cast<const float *>(qb + (int64_t)min(qr1, p.nq - 1) * p.q.nb[1]);
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const int c = ks * 16 + cq;
            qa[ks][0] = pack_h2(r0[c], r0[c + 1]);
            qa[ks][1] = pack_h2(r1[c], r1[c + 1]);
            qa[ks][2] = pack_h2(r0[c + 8], r0[c + 9]);
            qa[ks][3] = pack_h2(r1[c + 8], r1[c + 9]);
        }
    }
    float o[ND][4];
#pragma unroll
    for (int j = 0; j < ND; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;   // running maxima (base-2 domain) and sums

    const uint8_t *kb = k + (int64_t)hk * p.k.nb[2] + (int64_t)b * p.k.nb[3];
    const uint8_t *vb = v + (int64_t)hk * p.v.nb[2] + (int64_t)b * p.v.nb[3];
    const uint8_t *mb = mask ? mask + (int64_t)(h % p.m_ne2) * p.m.nb[2] + (int64_t)(b % p.m_ne3) * p.m.nb[3] : nullptr;
    const __half *mr0 = mb ? reinterpret_cast<const __half *>(mb + (int64_t)min(qr0, p.nq - 1) * p.m.nb[1]) : nullptr;
    const __half *mr1 = mb ? reinterpret_cast<const __half *>(mb + (int64_t)min(qr1, p.nq - 1) * p.m.nb[1]) : nullptr;
    const float LOG2E = 1.4426950408889634f;
    // ALiBi slope of this head (ggml_compute_forward_flash_attn_ext_f16: m0^(h+1) or m1^(2(h-n)+1)); 1 without a bias
    float slope = 1.f;
    if (p.max_bias > 0.f) slope = h < p.n_head_log2 ? powf(p.m0, (float)(h + 1)) : powf(p.m1, (float)(2 * (h - p.n_head_log2) + 1));

    for (int kt = k_begin; kt < k_end; kt += FA_KT) {
        // ---- this lane's mask values of the tile (2 rows x 16 keys); a tile that is -inf for every
        // query of the CTA (the upper triangle of a causal mask) is skipped before anything is loaded
        __half mk[FA_KT / 8][4];
        bool dead = mb != nullptr;
        if (mb) {
#pragma unroll
            for (int j = 0; j < FA_KT / 8; j++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = kt + j * 8 + cq + (e & 1);
                    const __half *mr = (e & 2) ? mr1 : mr0;
                    mk[j][e] = key < k_end ? mr[key] : __ushort_as_half(0xfc00);   // -inf past the last key
                    dead = dead && (__half_as_ushort(mk[j][e]) == 0xfc00);
                }
            }
        }
        if (__syncthreads_and(dead)) continue;   // also: the previous tile has been consumed
        for (int u = tid; u < FA_KT * (D / 8); u += FA_WARPS * 32) {
            const int row = u / (D / 8), c8 = u % (D / 8);
            const bool live = kt + row < k_end;
            const int64_t key = min(kt + row, k_end - 1);
            stage8<KF32>(Ks + row * LDS + c8 * 8, kb + key * p.k.nb[1] + c8 * 8 * (KF32 ? 4 : 2), live);
            stage8<VF32>(Vs + row * LDS + c8 * 8, vb + key * p.v.nb[1] + c8 * 8 * (VF32 ? 4 : 2), live);
        }
        __syncthreads();

        // ---- S = Q K^T for 64 keys: 8 n-tiles of 8 keys
        float s[FA_KT / 8][4];
#pragma unroll
        for (int j = 0; j < FA_KT / 8; j++) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            const __half *krow = Ks + (j * 8 + (lane >> 2)) * LDS + cq;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(krow + ks * 16);
                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(krow + ks * 16 + 8);
                mma16816(s[j], qa[ks], b0, b1);
            }
        }
        // ---- scale, soft cap, mask; scores move to the base-2 domain
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int j = 0; j < FA_KT / 8; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = kt + j * 8 + cq + (e & 1);
                float x = s[j][e] * p.scale;
                if (p.softcap != 0.f) x = p.softcap * tanhf(x);
                if (mb && key < k_end) x += slope * __half2float(mk[j][e]);
                x = key < k_end ? x * LOG2E : -CUDART_INF_F;
                s[j][e] = x;
                if (e & 2) mx1 = fmaxf(mx1, x);
                else mx0 = fmaxf(mx0, x);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // a row that has seen only masked keys keeps a finite reference so that exp2(-inf - ref) = 0
        const float ref0 = mx0 == -CUDART_INF_F ? 0.f : mx0, ref1 = mx1 == -CUDART_INF_F ? 0.f : mx1;
        const float a0 = exp2f(m0 - ref0), a1 = exp2f(m1 - ref1);   // m = -inf gives 0: nothing accumulated yet
        m0 = mx0;
        m1 = mx1;
        l0 *= a0;
        l1 *= a1;
#pragma unroll
        for (int j = 0; j < ND; j++) {
            o[j][0] *= a0; o[j][1] *= a0;
            o[j][2] *= a1; o[j][3] *= a1;
        }
        // ---- P = exp2(S - m) as A fragments; O += P V
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int t = 0; t < FA_KT / 16; t++) {
            uint32_t pa[4];
            float e00 = exp2f(s[2 * t][0] - ref0), e01 = exp2f(s[2 * t][1] - ref0);
            float e10 = exp2f(s[2 * t][2] - ref1), e11 = exp2f(s[2 * t][3] - ref1);
            float f00 = exp2f(s[2 * t + 1][0] - ref0), f01 = exp2f(s[2 * t + 1][1] - ref0);
            float f10 = exp2f(s[2 * t + 1][2] - ref1), f11 = exp2f(s[2 * t + 1][3] - ref1);
            ps0 += e00 + e01 + f00 + f01;
            ps1 += e10 + e11 + f10 + f11;
            pa[0] = pack_h2(e00, e01);
            pa[1] = pack_h2(e10, e11);
            pa[2] = pack_h2(f00, f01);
            pa[3] = pack_h2(f10, f11);
            const uint32_t vaddr = (uint32_t)__cvta_generic_to_shared(Vs + (t * 16 + (lane & 15)) * LDS);
#pragma unroll
            for (int j = 0; j < ND; j++) {
                uint32_t b0, b1;
                ldsm_x2_trans(b0, b1, vaddr + j * 16);
                mma16816(o[j], pa, b0, b1);
            }
        }
        l0 += ps0;
        l1 += ps1;
    }
    // ---- row sums across the quad, normalise, store [Dv, nh, nq, nb]
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (p.parts > 1) {
        // (maximum, sum, unnormalised output) of this stretch: [batch][head][query][part][D + 2]
        if (qr0 < p.nq) {
            float *d = partial + ((((int64_t)b * p.nh + h) * p.nq + qr0) * p.parts + part) * (D + 2);
            if (cq == 0) { d[0] = m0; d[1] = l0; }
#pragma unroll
            for (int j = 0; j < ND; j++) *reinterpret_cast<float2 *>(d + 2 + j * 8 + cq) = make_float2(o[j][0], o[j][1]);
        }
        if (qr1 < p.nq) {
            float *d = partial + ((((int64_t)b * p.nh + h) * p.nq + qr1) * p.parts + part) * (D + 2);
            if (cq == 0) { d[0] = m1; d[1] = l1; }
#pragma unroll
            for (int j = 0; j < ND; j++) *reinterpret_cast<float2 *>(d + 2 + j * 8 + cq) = make_float2(o[j][2], o[j][3]);
        }
        return;
    }
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (qr0 < p.nq) {
        float *d = out + (((int64_t)b * p.nq + qr0) * p.nh + h) * D;
#pragma unroll
        for (int j = 0; j < ND; j++) *reinterpret_cast<float2 *>(d + j * 8 + cq) = make_float2(o[j][0] * i0, o[j][1] * i0);
    }
    if (qr1 < p.nq) {
        float *d = out + (((int64_t)b * p.nq + qr1) * p.nh + h) * D;
#pragma unroll
        for (int j = 0; j < ND; j++) *reinterpret_cast<float2 *>(d + j * 8 + cq) = make_float2(o[j][2] * i1, o[j][3] * i1);
    }
}

// merges the stretches of a split: one CTA per (query, head, batch), one thread per output element
template <int D>
__global__ void __launch_bounds__(D) k_flash_merge(FlashArgs p, const float *__restrict__ partial, float *__restrict__ out) {
    griddep_launch();
    griddep_wait();
    const int q = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    const float *pp = partial + (((int64_t)b * p.nh + h) * p.nq + q) * p.parts * (D + 2);
    float m = -CUDART_INF_F;
    for (int c = 0; c < p.parts; c++) m = fmaxf(m, pp[(int64_t)c * (D + 2)]);
    const float ref = m == -CUDART_INF_F ? 0.f : m;
    float l = 0.f, a = 0.f;
    for (int c = 0; c < p.parts; c++) {
        const float f = exp2f(pp[(int64_t)c * (D + 2)] - ref);   // a stretch that saw only masked keys has m = -inf: weight 0
        l += pp[(int64_t)c * (D + 2) + 1] * f;
        a += pp[(int64_t)c * (D + 2) + 2 + d] * f;
    }
    out[(((int64_t)b * p.nq + q) * p.nh + h) * D + d] = l > 0.f ? a / l : 0.f;
}

// ---------------------------------------------------------------- any other head size
// Head sizes other than 64 / 128, up to 512, keys and values of different sizes included (the reference takes any value
// head size up to 512, crates/kernels/src/cuda/lower.rs:594-596; its tests run 72, 80, 96, 112 and 256,
// crates/tensorlisp/tests/native.rs:283-346): one CTA per (query, stretch of keys, head, batch) as in the reference's
// fa_main / fa_split, a warp per key in turn, lane i holding elements i, i + 32, ... of the rows; f32 dot product,
// online softmax and accumulation per warp, the warps merged through shared memory. With an f16 cache the query is
// rounded to f16 first, as the CPU backend does. Not a tuned kernel.
constexpr int FA_ANY_MAX = 512, FA_ANY_PER_LANE = FA_ANY_MAX / 32;

// element e of a key or value row: MODE 0 = f16, 1 = f32, 2 = any other type the executor decodes (bf16 and the block types)
template <int MODE>
__device__ __forceinline__ float fa_any_elem(const uint8_t *row, uint32_t ty, int e) {
    if (MODE == 0) return __half2float(reinterpret_cast<const __half *>(row)[e]);
    if (MODE == 1) return reinterpret_cast<const float *>(row)[e];
    return is_quant(ty) ? dq_elem(row, ty, e) : ld_elem(row + (int64_t)e * 2, ty);   // the only other plain type here is bf16
}

template <int KM, int VM>
__global__ void __launch_bounds__(FA_WARPS * 32) k_flash_attn_any(FlashArgs p, const uint8_t *__restrict__ q, const uint8_t *__restrict__ k,
                                                                  const uint8_t *__restrict__ v, const uint8_t *__restrict__ mask,
                                                                  float *__restrict__ out, float *__restrict__ partial) {
    griddep_launch();
    griddep_wait();
    __shared__ float ml[FA_WARPS][2];
    __shared__ float accs[FA_WARPS][FA_ANY_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = blockIdx.x % p.parts, qi = blockIdx.x / p.parts;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / (p.nh / p.nhkv);
    const int k_begin = part * p.part_len, k_end = min(p.nkv, k_begin + p.part_len);
    const int D = p.d, DV = p.dv;
    float qf[FA_ANY_PER_LANE], acc[FA_ANY_PER_LANE];
    {
        const float *qr = reinterpret_cast<const float *>(q + (int64_t)qi * p.q.nb[1] + (int64_t)h * p.q.nb[2] + (int64_t)b * p.q.nb[3]);
#pragma unroll
        for (int j = 0; j < FA_ANY_PER_LANE; j++) {
            const int e = lane + 32 * j;
            float x = e < D ? qr[e] : 0.f;
            if (KM == 0) x = __half2float(__float2half_rn(x));
            qf[j] = x;
            acc[j] = 0.f;
        }
    }
    const uint8_t *kb = k + (int64_t)hk * p.k.nb[2] + (int64_t)b * p.k.nb[3];
    const uint8_t *vb = v + (int64_t)hk * p.v.nb[2] + (int64_t)b * p.v.nb[3];
    const __half *mr = mask ? reinterpret_cast<const __half *>(mask + (int64_t)(h % p.m_ne2) * p.m.nb[2] + (int64_t)(b % p.m_ne3) * p.m.nb[3] +
                                                               (int64_t)qi * p.m.nb[1])
                            : nullptr;
    const float LOG2E = 1.4426950408889634f;
    float slope = 1.f;
    if (p.max_bias > 0.f) slope = h < p.n_head_log2 ? powf(p.m0, (float)(h + 1)) : powf(p.m1, (float)(2 * (h - p.n_head_log2) + 1));
    float m_run = -CUDART_INF_F, l_run = 0.f;
    for (int key = k_begin + warp; key < k_end; key += FA_WARPS) {
        float mv = 0.f;
        if (mr) {
            const __half mh = mr[key];
            if (__half_as_ushort(mh) == 0xfc00) continue;   // a key masked with -inf takes no part
            mv = slope * __half2float(mh);
        }
        const uint8_t *kr = kb + (int64_t)key * p.k.nb[1];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < FA_ANY_PER_LANE; j++) {
            const int e = lane + 32 * j;
            if (32 * j < D && e < D)
                dot = fmaf(qf[j], fa_any_elem<KM>(kr, p.k_ty, e), dot);
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sh);
        float x = dot * p.scale;
        if (p.softcap != 0.f) x = p.softcap * tanhf(x);
        x = (x + mv) * LOG2E;
        if (x == -CUDART_INF_F) continue;
        const float m_new = fmaxf(m_run, x);
        const float corr = exp2f(m_run - m_new), pw = exp2f(x - m_new);
        m_run = m_new;
        l_run = l_run * corr + pw;
        const uint8_t *vr = vb + (int64_t)key * p.v.nb[1];
#pragma unroll
        for (int j = 0; j < FA_ANY_PER_LANE; j++) {
            const int e = lane + 32 * j;
            if (32 * j < DV && e < DV)
                acc[j] = fmaf(pw, fa_any_elem<VM>(vr, p.v_ty, e), acc[j] * corr);
        }
    }
    if (lane == 0) {
        ml[warp][0] = m_run;
        ml[warp][1] = l_run;
    }
#pragma unroll
    for (int j = 0; j < FA_ANY_PER_LANE; j++) {
        const int e = lane + 32 * j;
        if (e < DV) accs[warp][e] = acc[j];
    }
    __syncthreads();
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < FA_WARPS; w++) m = fmaxf(m, ml[w][0]);
    const float ref = m == -CUDART_INF_F ? 0.f : m;
    float f[FA_WARPS], l = 0.f;
#pragma unroll
    for (int w = 0; w < FA_WARPS; w++) {
        f[w] = exp2f(ml[w][0] - ref);   // a warp that saw no live key has m = -inf: weight 0
        l += ml[w][1] * f[w];
    }
    float *pp = p.parts > 1 ? partial + ((((int64_t)b * p.nh + h) * p.nq + qi) * p.parts + part) * (DV + 2) : nullptr;
    float *o = out + (((int64_t)b * p.nq + qi) * p.nh + h) * DV;
    if (pp && threadIdx.x == 0) {
        pp[0] = m;
        pp[1] = l;
    }
    for (int d = threadIdx.x; d < DV; d += FA_WARPS * 32) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < FA_WARPS; w++) a += accs[w][d] * f[w];
        if (pp) pp[2 + d] = a;
        else o[d] = l > 0.f ? a / l : 0.f;
    }
}

// merges the stretches of a split for any value head size: one CTA per (query, head, batch)
__global__ void __launch_bounds__(128) k_flash_merge_any(FlashArgs p, const float *__restrict__ partial, float *__restrict__ out) {
    griddep_launch();
    griddep_wait();
    const int q = blockIdx.x, h = blockIdx.y, b = blockIdx.z, DV = p.dv;
    const float *pp = partial + (((int64_t)b * p.nh + h) * p.nq + q) * p.parts * (DV + 2);
    float m = -CUDART_INF_F;
    for (int c = 0; c < p.parts; c++) m = fmaxf(m, pp[(int64_t)c * (DV + 2)]);
    const float ref = m == -CUDART_INF_F ? 0.f : m;
    float l = 0.f;
    for (int c = 0; c < p.parts; c++) l += pp[(int64_t)c * (DV + 2) + 1] * exp2f(pp[(int64_t)c * (DV + 2)] - ref);
    for (int d = threadIdx.x; d < DV; d += 128) {
        float a = 0.f;
        for (int c = 0; c < p.parts; c++) a += pp[(int64_t)c * (DV + 2) + 2 + d] * exp2f(pp[(int64_t)c * (DV + 2)] - ref);
        out[(((int64_t)b * p.nq + q) * p.nh + h) * DV + d] = l > 0.f ? a / l : 0.f;
    }
}

}  // namespace

static bool fa_tensor_core_size(int64_t d, int64_t dv) { return d == dv && (d == 64 || d == 128); }
static bool fa_tensor_core(const FlashArgs &p) {
    return fa_tensor_core_size(p.d, p.dv) && (p.k_ty == TLB_TYPE_F16 || p.k_ty == TLB_TYPE_F32) && (p.v_ty == TLB_TYPE_F16 || p.v_ty == TLB_TYPE_F32);
}
bool flash_supported(int64_t d, int64_t dv) { return d >= 1 && dv >= 1 && d <= FA_ANY_MAX && dv <= FA_ANY_MAX; }
bool flash_rows_need_alignment(int64_t d, int64_t dv) { return fa_tensor_core_size(d, dv); }

// Split-KV for few queries over a long dense cache (the reference's rule, crates/kernels/src/cuda/lower.rs:764-779, on
// this kernel's 64-key tiles): without it a one-query node runs heads x batch CTAs whatever the length of the cache.
void flash_split_plan(FlashArgs &p, int sm_count) {
    p.part_len = p.nkv > 0 ? p.nkv : 1;
    p.parts = 1;
    const char *e = getenv("TL_NATIVE_FA");
    const bool tc = fa_tensor_core(p);
    // the other head sizes run one query per CTA, like the reference: its rule as it stands (one query, 256 keys or more)
    if (p.nq > (tc ? FA_QT : 1) || p.nkv < 256 || (e && std::string(e) == "plain")) return;
    const int64_t blocks = (int64_t)p.nh * p.nb;
    const int64_t want = ((int64_t)p.nkv * blocks + 4 * (int64_t)sm_count - 1) / (4 * (int64_t)sm_count);
    const int64_t part_len = std::max<int64_t>(FA_KT, (want + FA_KT - 1) / FA_KT * FA_KT);
    const int64_t parts = (p.nkv + part_len - 1) / part_len;
    if (parts >= 2) {
        p.part_len = (int)part_len;
        p.parts = (int)parts;
    }
}
uint64_t flash_split_scratch_bytes(const FlashArgs &p) {
    return p.parts > 1 ? (uint64_t)p.nb * p.nh * p.nq * p.parts * (p.dv + 2) * 4 : 0;
}

template <int D>
static cudaError_t launch_fa(const FlashArgs &p, const void *q, const void *k, const void *v, const void *mask, float *out, float *partial,
                             cudaStream_t st) {
    const dim3 grid((unsigned)((p.nq + FA_QT - 1) / FA_QT * p.parts), (unsigned)p.nh, (unsigned)p.nb), block(FA_WARPS * 32);
    const uint8_t *q8 = (const uint8_t *)q, *k8 = (const uint8_t *)k, *v8 = (const uint8_t *)v, *m8 = (const uint8_t *)mask;
    cudaError_t e;
    if (p.k_f32 && p.v_f32) e = launch_pdl(k_flash_attn<D, true, true>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else if (p.k_f32) e = launch_pdl(k_flash_attn<D, true, false>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else if (p.v_f32) e = launch_pdl(k_flash_attn<D, false, true>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else e = launch_pdl(k_flash_attn<D, false, false>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    if (e == cudaSuccess && p.parts > 1)
        e = launch_pdl(k_flash_merge<D>, dim3((unsigned)p.nq, (unsigned)p.nh, (unsigned)p.nb), dim3(D), 0, st, p, (const float *)partial, out);
    return e;
}

cudaError_t launch_flash_attn(const FlashArgs &p, const void *q, const void *k, const void *v, const void *mask, float *out, void *scratch,
                              cudaStream_t st) {
    if (p.nq == 0 || p.nh == 0 || p.nb == 0) return cudaSuccess;
    if (p.parts < 1 || (p.parts > 1 && !scratch)) return cudaErrorInvalidValue;
    if (fa_tensor_core(p))
        return p.d == 64 ? launch_fa<64>(p, q, k, v, mask, out, (float *)scratch, st) : launch_fa<128>(p, q, k, v, mask, out, (float *)scratch, st);
    if (!flash_supported(p.d, p.dv)) return cudaErrorInvalidValue;
    const dim3 grid((unsigned)(p.nq * p.parts), (unsigned)p.nh, (unsigned)p.nb), block(FA_WARPS * 32);
    const uint8_t *q8 = (const uint8_t *)q, *k8 = (const uint8_t *)k, *v8 = (const uint8_t *)v, *m8 = (const uint8_t *)mask;
    float *partial = (float *)scratch;
    cudaError_t e;
    const auto plain = [](uint32_t ty) { return ty == TLB_TYPE_F16 || ty == TLB_TYPE_F32; };
    if (!plain(p.k_ty) || !plain(p.v_ty)) e = launch_pdl(k_flash_attn_any<2, 2>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else if (p.k_f32 && p.v_f32) e = launch_pdl(k_flash_attn_any<1, 1>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else if (p.k_f32) e = launch_pdl(k_flash_attn_any<1, 0>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else if (p.v_f32) e = launch_pdl(k_flash_attn_any<0, 1>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    else e = launch_pdl(k_flash_attn_any<0, 0>, grid, block, 0, st, p, q8, k8, v8, m8, out, partial);
    if (e == cudaSuccess && p.parts > 1)
        e = launch_pdl(k_flash_merge_any, dim3((unsigned)p.nq, (unsigned)p.nh, (unsigned)p.nb), dim3(128), 0, st, p, (const float *)partial, out);
    return e;
}

}  // namespace tlb
