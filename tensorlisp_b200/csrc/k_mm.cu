// MUL_MAT with GGUF block-quantized weights (reference: crates/kernels/src/cuda/lower.rs:543-571 and
// native/mm.cu, whose semantics are y[m,n] = sum_k dq(W[k,m]) x[k,n]).
//
// Arithmetic follows the reference's CPU backend exactly (ggml-cpu.c:1272-1357): the activations
// have already been quantized to int8 blocks (k_quant.cu), each output is an integer dot product
// per block scaled in f32 (ggml-cpu/quants.c:451-479 for Q8_0, :225-260 for Q4_0, :696-770 for
// Q4_K). Only the order of the f32 additions differs.
//
// k_gemv_stream: persistent CTAs stream tiles of whole weight rows (rows are contiguous, so a
// tile is one contiguous byte range) into shared memory with 1-D bulk copies (cp.async.bulk +
// mbarrier) through a multi-stage ring, so tens of KB per SM are always in flight without
// spending registers or issue slots; warps then take 128-bit pieces of a super-block out of
// shared memory, unpack nibbles in registers, and use dp4a against the int8 activations.
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "kernels.h"

namespace tlb {

// ---------------------------------------------------------------- mbarrier / bulk-copy helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: gives up after `limit` polls and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    const uint32_t a = smem_u32(bar);
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_STAGES = 4;
constexpr int GEMV_STAGE_BYTES = 40 * 1024;  // tile of whole rows, at most this many bytes
constexpr int GEMV_PAD = 16;                 // word-aligned reads may run 2 bytes past a block

// ---------------------------------------------------------------- per-row dot products from shared memory
template <int NC>
__device__ __forceinline__ void row_q4_K(const uint8_t *row, int64_t K, const int8_t *aq, const float *ad,
                                         const int16_t *ab, int n0, int lane, int part, int wpr, float (&f)[NC]) {
    const int piece = lane & 7, c = piece >> 1, half = piece & 1;
    const int nsb = (int)(K / 256);
    for (int sb = (lane >> 3) + 4 * part; sb < nsb; sb += 4 * wpr) {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(row + sb * 144);
        const uint4 q = *reinterpret_cast<const uint4 *>(row + sb * 144 + 16 + 16 * piece);
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        // 6-bit scales/mins of sub-blocks 2c and 2c+1 (get_scale_min_k4, ggml-quants.c:880-887)
        const int sh = (c & 1) * 16;
        const uint32_t a16 = (hdr.y >> sh) & 0xffffu, b16 = (hdr.z >> sh) & 0xffffu, c16 = (hdr.w >> sh) & 0xffffu;
        uint32_t sc2, m2;
        if (c < 2) {
            sc2 = a16 & 0x3f3fu;
            m2 = b16 & 0x3f3fu;
        } else {
            sc2 = (c16 & 0x0f0fu) | ((a16 >> 2) & 0x3030u);
            m2 = ((c16 >> 4) & 0x0f0fu) | ((b16 >> 2) & 0x3030u);
        }
        const int sc_lo = sc2 & 0xff, sc_hi = sc2 >> 8, m_lo = m2 & 0xff, m_hi = m2 >> 8;
        const uint32_t lo[4] = {q.x & 0x0f0f0f0fu, q.y & 0x0f0f0f0fu, q.z & 0x0f0f0f0fu, q.w & 0x0f0f0f0fu};
        const uint32_t hi[4] = {(q.x >> 4) & 0x0f0f0f0fu, (q.y >> 4) & 0x0f0f0f0fu, (q.z >> 4) & 0x0f0f0f0fu,
                                (q.w >> 4) & 0x0f0f0f0fu};
        const int64_t kbase = (int64_t)sb * 256 + c * 64 + half * 16;
#pragma unroll
        for (int n = 0; n < NC; n++) {
            const int8_t *a = aq + (int64_t)(n0 + n) * K + kbase;
            const int4 al = *reinterpret_cast<const int4 *>(a);
            const int4 ah = *reinterpret_cast<const int4 *>(a + 32);
            int il = __dp4a((int)lo[0], al.x, 0);
            il = __dp4a((int)lo[1], al.y, il);
            il = __dp4a((int)lo[2], al.z, il);
            il = __dp4a((int)lo[3], al.w, il);
            int ih = __dp4a((int)hi[0], ah.x, 0);
            ih = __dp4a((int)hi[1], ah.y, ih);
            ih = __dp4a((int)hi[2], ah.z, ih);
            ih = __dp4a((int)hi[3], ah.w, ih);
            const int16_t *bs = ab + (int64_t)(n0 + n) * (K / 16) + sb * 16 + 4 * c + half;
            const int acc = sc_lo * il + sc_hi * ih;
            const int macc = m_lo * (int)bs[0] + m_hi * (int)bs[2];
            const float yd = ad[(int64_t)(n0 + n) * (K / 256) + sb];
            f[n] += yd * (dm.x * (float)acc - dm.y * (float)macc);
        }
    }
}

// 34-byte / 18-byte blocks are only 2-byte aligned: read whole words and realign by 16 bits.
template <int NC>
__device__ __forceinline__ void row_q8_0(const uint8_t *row, int64_t K, const int8_t *aq, const float *ad, int n0,
                                         int lane, int part, int wpr, float (&f)[NC]) {
    const int nblk = (int)(K / 32);
    for (int b = lane + 32 * part; b < nblk; b += 32 * wpr) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(row + ((34 * b) & ~3));
        uint32_t r[9];
#pragma unroll
        for (int i = 0; i < 9; i++) r[i] = w[i];
        uint32_t qs[8];
        uint16_t dh;
        if (b & 1) {
            dh = (uint16_t)(r[0] >> 16);
#pragma unroll
            for (int i = 0; i < 8; i++) qs[i] = r[i + 1];
        } else {
            dh = (uint16_t)(r[0] & 0xffffu);
#pragma unroll
            for (int i = 0; i < 8; i++) qs[i] = __funnelshift_r(r[i], r[i + 1], 16);
        }
        const float d = __half2float(__ushort_as_half(dh));
#pragma unroll
        for (int n = 0; n < NC; n++) {
            const int4 *a = reinterpret_cast<const int4 *>(aq + (int64_t)(n0 + n) * K + (int64_t)b * 32);
            const int4 a0 = a[0], a1 = a[1];
            int s = __dp4a((int)qs[0], a0.x, 0);
            s = __dp4a((int)qs[1], a0.y, s);
            s = __dp4a((int)qs[2], a0.z, s);
            s = __dp4a((int)qs[3], a0.w, s);
            s = __dp4a((int)qs[4], a1.x, s);
            s = __dp4a((int)qs[5], a1.y, s);
            s = __dp4a((int)qs[6], a1.z, s);
            s = __dp4a((int)qs[7], a1.w, s);
            f[n] += (float)s * (d * ad[(int64_t)(n0 + n) * (K / 32) + b]);
        }
    }
}

template <int NC>
__device__ __forceinline__ void row_q4_0(const uint8_t *row, int64_t K, const int8_t *aq, const float *ad, int n0,
                                         int lane, int part, int wpr, float (&f)[NC]) {
    const int nblk = (int)(K / 32);
    for (int b = lane + 32 * part; b < nblk; b += 32 * wpr) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(row + ((18 * b) & ~3));
        uint32_t r[5];
#pragma unroll
        for (int i = 0; i < 5; i++) r[i] = w[i];
        uint32_t qs[4];
        uint16_t dh;
        if (b & 1) {
            dh = (uint16_t)(r[0] >> 16);
#pragma unroll
            for (int i = 0; i < 4; i++) qs[i] = r[i + 1];
        } else {
            dh = (uint16_t)(r[0] & 0xffffu);
#pragma unroll
            for (int i = 0; i < 4; i++) qs[i] = __funnelshift_r(r[i], r[i + 1], 16);
        }
        const float d = __half2float(__ushort_as_half(dh));
#pragma unroll
        for (int n = 0; n < NC; n++) {
            const int4 *a = reinterpret_cast<const int4 *>(aq + (int64_t)(n0 + n) * K + (int64_t)b * 32);
            const int4 a0 = a[0], a1 = a[1];
            const int av0[4] = {a0.x, a0.y, a0.z, a0.w}, av1[4] = {a1.x, a1.y, a1.z, a1.w};
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int lo = (int)__vsub4(qs[i] & 0x0f0f0f0fu, 0x08080808u);
                const int hi = (int)__vsub4((qs[i] >> 4) & 0x0f0f0f0fu, 0x08080808u);
                s = __dp4a(lo, av0[i], s);
                s = __dp4a(hi, av1[i], s);
            }
            f[n] += (float)s * d * ad[(int64_t)(n0 + n) * (K / 32) + b];
        }
    }
}

// ---------------------------------------------------------------- the streaming kernel
template <int TYPE, int NC>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
k_gemv_stream(const uint8_t *__restrict__ W, int64_t row_bytes, int64_t M, int64_t K, const int8_t *__restrict__ aq,
              const float *__restrict__ ad, const int16_t *__restrict__ ab, float *__restrict__ y, int64_t ldy, int n0,
              int rows_per_tile, int wpr, int stage_stride, int *__restrict__ err) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full[GEMV_STAGES];
    __shared__ int s_fail;
    __shared__ float partial[2][GEMV_WARPS][NC];
    int pbuf = 0;
    const int rows_per_pass = GEMV_WARPS / wpr;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t n_tiles = (M + rows_per_tile - 1) / rows_per_tile;
    const int64_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    if (tid == 0) {
        for (int s = 0; s < GEMV_STAGES; s++) mbar_init(&full[s], 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](int64_t i) {  // tile i of this CTA -> stage i % STAGES
        const int64_t tile = blockIdx.x + i * gridDim.x;
        const int64_t r0 = tile * rows_per_tile;
        const int64_t rows = min((int64_t)rows_per_tile, M - r0);
        const uint32_t bytes = (uint32_t)(rows * row_bytes);
        const int s = (int)(i % GEMV_STAGES);
        mbar_expect_tx(&full[s], bytes);
        bulk_g2s(smem + (size_t)s * stage_stride, W + r0 * row_bytes, bytes, &full[s]);
    };
    if (tid == 0)
        for (int64_t i = 0; i < my_tiles && i < GEMV_STAGES; i++) issue(i);

    int64_t issued = my_tiles < GEMV_STAGES ? my_tiles : GEMV_STAGES;
    int64_t done = 0;
    for (int64_t i = 0; i < my_tiles; i++) {
        const int s = (int)(i % GEMV_STAGES);
        const bool ok = !__syncthreads_or(!mbar_wait(&full[s], (uint32_t)((i / GEMV_STAGES) & 1)));  // uniform
        if (!ok) {
            if (tid == 0) s_fail = 1;
            __syncthreads();
            break;
        }
        const int64_t tile = blockIdx.x + i * gridDim.x;
        const int64_t r0 = tile * rows_per_tile;
        const int rows = (int)min((int64_t)rows_per_tile, M - r0);
        if (ok) {
            const uint8_t *base = smem + (size_t)s * stage_stride;
            for (int rb = 0; rb < rows; rb += rows_per_pass) {
                const int r = rb + warp / wpr, part = warp % wpr;
                float f[NC];
#pragma unroll
                for (int n = 0; n < NC; n++) f[n] = 0.f;
                if (r < rows) {
                    const uint8_t *row = base + (size_t)r * row_bytes;
                    if (TYPE == TLB_TYPE_Q4_K) row_q4_K<NC>(row, K, aq, ad, ab, n0, lane, part, wpr, f);
                    else if (TYPE == TLB_TYPE_Q8_0) row_q8_0<NC>(row, K, aq, ad, n0, lane, part, wpr, f);
                    else row_q4_0<NC>(row, K, aq, ad, n0, lane, part, wpr, f);
                }
#pragma unroll
                for (int n = 0; n < NC; n++) f[n] = warp_sum(f[n]);
                if (wpr == 1) {
                    if (lane == 0 && r < rows) {
#pragma unroll
                        for (int n = 0; n < NC; n++) y[(int64_t)(n0 + n) * ldy + r0 + r] = f[n];
                    }
                } else {
                    // several warps share a row: combine their partial sums through shared memory
                    if (lane == 0) {
#pragma unroll
                        for (int n = 0; n < NC; n++) partial[pbuf][warp][n] = f[n];
                    }
                    __syncthreads();
                    if (tid < rows_per_pass * NC) {
                        const int rr = tid / NC, n = tid % NC;
                        if (rb + rr < rows) {
                            float v = 0.f;
                            for (int pp = 0; pp < wpr; pp++) v += partial[pbuf][rr * wpr + pp][n];
                            y[(int64_t)(n0 + n) * ldy + r0 + rb + rr] = v;
                        }
                    }
                    pbuf ^= 1;
                }
            }
        }
        __syncthreads();  // every warp is done with stage s
        done = i + 1;
        if (tid == 0 && i + GEMV_STAGES < my_tiles) {
            issue(i + GEMV_STAGES);
            issued = i + GEMV_STAGES + 1;
        }
    }
    if (s_fail && tid == 0) {
        // wait (bounded) for the copies still in flight before the CTA's shared memory is released
        for (int64_t j = done; j < issued; j++) mbar_wait(&full[j % GEMV_STAGES], (uint32_t)((j / GEMV_STAGES) & 1));
        atomicExch(err, 1);
    }
}

bool gemv_supported(uint32_t type, int64_t K, int64_t M, int64_t N) {
    if (type != TLB_TYPE_Q4_K && type != TLB_TYPE_Q8_0 && type != TLB_TYPE_Q4_0) return false;
    if (K % 256 != 0 || M < 1 || N < 1) return false;
    const int64_t rb = (int64_t)tlb_row_size(type, K);
    return rb % 16 == 0 && rb + GEMV_PAD <= GEMV_STAGE_BYTES;
}

template <int TYPE, int NC>
static void set_attr() {
    cudaFuncSetAttribute(k_gemv_stream<TYPE, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         GEMV_STAGES * (GEMV_STAGE_BYTES + 128));
}
template <int TYPE>
static void set_attr_type() {
    set_attr<TYPE, 1>(); set_attr<TYPE, 2>(); set_attr<TYPE, 3>(); set_attr<TYPE, 4>();
}
void gemv_configure() {
    set_attr_type<TLB_TYPE_Q4_K>();
    set_attr_type<TLB_TYPE_Q8_0>();
    set_attr_type<TLB_TYPE_Q4_0>();
}

template <int TYPE>
static cudaError_t launch_gemv_t(const void *W, int64_t K, int64_t M, const ActLayout &a, const void *act, float *y,
                                 int64_t ldy, int sm_count, int *err, cudaStream_t st) {
    const int64_t rb = (int64_t)tlb_row_size(TYPE, K);
    int rows_per_tile = (int)((GEMV_STAGE_BYTES - GEMV_PAD) / rb);
    // keep every SM busy: no more rows per tile than gives each SM a few tiles
    const int64_t want_tiles = (int64_t)sm_count * 4;
    const int64_t cap = (M + want_tiles - 1) / want_tiles;
    if (rows_per_tile > cap) rows_per_tile = (int)(cap < 1 ? 1 : cap);
    // whole warps' worth of rows keeps the 8 warps evenly loaded; with fewer rows than warps,
    // several warps share a row
    if (rows_per_tile > GEMV_WARPS) rows_per_tile = rows_per_tile / GEMV_WARPS * GEMV_WARPS;
    int wpr = 1;
    while (wpr * 2 * rows_per_tile <= GEMV_WARPS) wpr *= 2;
    const int64_t units = TYPE == TLB_TYPE_Q4_K ? K / 256 / 4 : K / 32 / 32;  // loop trips of one warp
    while (wpr > 1 && units < wpr) wpr /= 2;
    const int stage_stride = (int)(((int64_t)rows_per_tile * rb + GEMV_PAD + 127) / 128 * 128);
    const int64_t n_tiles = (M + rows_per_tile - 1) / rows_per_tile;
    const int grid = (int)(n_tiles < sm_count ? n_tiles : sm_count);
    const size_t smem = (size_t)GEMV_STAGES * stage_stride;
    const char *ab = (const char *)act;
    const int8_t *aq = (const int8_t *)(ab + a.qs_off);
    const float *ad = (const float *)(ab + a.d_off);
    const int16_t *bs = (const int16_t *)(ab + a.bsum_off);
    for (int n0 = 0; n0 < a.N;) {
        const int nc = (int)(a.N - n0 >= 4 ? 4 : a.N - n0);
#define GO(NCV)                                                                                                   \
    k_gemv_stream<TYPE, NCV><<<grid, GEMV_THREADS, smem, st>>>((const uint8_t *)W, rb, M, K, aq, ad, bs, y, ldy, n0, \
                                                              rows_per_tile, wpr, stage_stride, err)
        switch (nc) {
            case 1: GO(1); break;
            case 2: GO(2); break;
            case 3: GO(3); break;
            default: GO(4); break;
        }
#undef GO
        n0 += nc;
    }
    return cudaGetLastError();
}

cudaError_t launch_gemv(uint32_t type, const void *W, int64_t K, int64_t M, const ActLayout &a, const void *act,
                        float *y, int64_t ldy, int sm_count, int *err, cudaStream_t st) {
    switch (type) {
        case TLB_TYPE_Q4_K: return launch_gemv_t<TLB_TYPE_Q4_K>(W, K, M, a, act, y, ldy, sm_count, err, st);
        case TLB_TYPE_Q8_0: return launch_gemv_t<TLB_TYPE_Q8_0>(W, K, M, a, act, y, ldy, sm_count, err, st);
        case TLB_TYPE_Q4_0: return launch_gemv_t<TLB_TYPE_Q4_0>(W, K, M, a, act, y, ldy, sm_count, err, st);
        default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------- generic strided / batched product
// One warp per output element; lanes walk the row's blocks. Handles every shape the streaming
// kernel does not (K not a multiple of 256, strided or broadcast batches, plain weight types).
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &d, int &m) {
    if (j < 4) {
        d = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

__global__ void __launch_bounds__(128) k_mm_generic(MMGeneric p, const uint8_t *__restrict__ W, const uint8_t *__restrict__ X,
                                                     uint8_t *__restrict__ Y) {
    const int lane = threadIdx.x & 31;
    const int64_t m = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t M = p.y.ne[0], N = p.y.ne[1], K = p.w.ne[0];
    if (m >= M) return;
    const int64_t n = blockIdx.y % N, i2 = (blockIdx.y / N) % p.y.ne[2], i3 = blockIdx.z;
    const uint8_t *wrow = W + m * p.w.nb[1] + (i2 / p.r2) * p.w.nb[2] + (i3 / p.r3) * p.w.nb[3];
    float f = 0.f;
    if (p.wtype == TLB_TYPE_F32 || p.wtype == TLB_TYPE_F16 || p.wtype == TLB_TYPE_BF16) {
        const uint8_t *xcol = X + n * p.x.nb[1] + i2 * p.x.nb[2] + i3 * p.x.nb[3];
        for (int64_t k = lane; k < K; k += 32) {
            float wv;
            if (p.wtype == TLB_TYPE_F32) wv = reinterpret_cast<const float *>(wrow)[k];
            else if (p.wtype == TLB_TYPE_F16) wv = __half2float(reinterpret_cast<const __half *>(wrow)[k]);
            else wv = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(wrow)[k]);
            f += wv * *reinterpret_cast<const float *>(xcol + k * p.x.nb[0]);
        }
    } else {
        const int64_t col = n + N * (i2 + p.y.ne[2] * i3);  // column of the quantized activation block
        const char *ab = (const char *)p.act;
        const int8_t *aq = (const int8_t *)(ab + p.a.qs_off) + col * K;
        const float *ad = (const float *)(ab + p.a.d_off);
        if (p.wtype == TLB_TYPE_Q8_0) {
            for (int64_t b = lane; b < K / 32; b += 32) {
                const uint8_t *blk = wrow + b * 34;
                const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk)));
                const int8_t *qs = reinterpret_cast<const int8_t *>(blk + 2);
                int s = 0;
                for (int j = 0; j < 32; j++) s += (int)qs[j] * (int)aq[b * 32 + j];
                f += (float)s * (d * ad[col * (K / 32) + b]);
            }
        } else if (p.wtype == TLB_TYPE_Q4_0) {
            for (int64_t b = lane; b < K / 32; b += 32) {
                const uint8_t *blk = wrow + b * 18;
                const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk)));
                int s = 0;
                for (int j = 0; j < 16; j++) {
                    s += ((int)(blk[2 + j] & 0x0F) - 8) * (int)aq[b * 32 + j];
                    s += ((int)(blk[2 + j] >> 4) - 8) * (int)aq[b * 32 + j + 16];
                }
                f += (float)s * d * ad[col * (K / 32) + b];
            }
        } else {  // Q4_K, one (super-block, sub-block) per lane step
            const int16_t *bs = (const int16_t *)(ab + p.a.bsum_off) + col * (K / 16);
            for (int64_t u = lane; u < K / 32; u += 32) {
                const int64_t sb = u >> 3;
                const int j = (int)(u & 7);
                const uint8_t *blk = wrow + sb * 144;
                const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk)));
                const float dmin = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(blk + 2)));
                int sc, mn;
                scale_min_k4(j, blk + 4, sc, mn);
                const uint8_t *q = blk + 16 + (j >> 1) * 32;
                const int shift = (j & 1) * 4;
                int s = 0;
                for (int l = 0; l < 32; l++) s += (int)((q[l] >> shift) & 0xF) * (int)aq[sb * 256 + j * 32 + l];
                const int bsum = (int)bs[sb * 16 + 2 * j] + (int)bs[sb * 16 + 2 * j + 1];
                f += ad[col * (K / 256) + sb] * (d * (float)(sc * s) - dmin * (float)(mn * bsum));
            }
        }
    }
    f = warp_sum(f);
    if (lane == 0) *reinterpret_cast<float *>(Y + m * p.y.nb[0] + n * p.y.nb[1] + i2 * p.y.nb[2] + i3 * p.y.nb[3]) = f;
}

cudaError_t launch_mm_generic(const MMGeneric &p, const void *W, const void *X, void *Y, cudaStream_t st) {
    const int64_t M = p.y.ne[0], N = p.y.ne[1];
    if (M == 0 || N == 0) return cudaSuccess;
    dim3 grid((unsigned)((M + 3) / 4), (unsigned)(N * p.y.ne[2]), (unsigned)p.y.ne[3]);
    k_mm_generic<<<grid, 128, 0, st>>>(p, (const uint8_t *)W, (const uint8_t *)X, (uint8_t *)Y);
    return cudaGetLastError();
}

}  // namespace tlb
