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
#include <algorithm>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "kernels.h"
#include "dequant.cuh"
#include "pdl.cuh"

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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 19)) {   // about two seconds: a probe of an incomplete phase takes about 4 us
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

constexpr int GEMV_CW = 16;                       // consumer warps
constexpr int GEMV_THREADS = 32 * (GEMV_CW + 1);  // plus one warp whose lane 0 issues the bulk copies
constexpr int GEMV_STAGES = 4;                    // power of two
constexpr int GEMV_STAGE_BYTES = 40 * 1024;       // tile of whole rows, at most this many bytes
constexpr int GEMV_PAD = 16;                      // word-aligned reads may run 2 bytes past a block
constexpr int GEMV_ACT_SMEM = 60 * 1024;          // Q4_K: int8 activation codes of one pass, staged in shared memory

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// unsigned bytes x signed bytes
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Shared-memory order of one column's int8 codes for the Q4_K kernel: a warp iteration covers 8
// super-blocks = 32 chunks of 64 codes (lane = chunk); the j-th 16-byte piece of every chunk of an
// iteration is contiguous in lane order, so each of a lane's four 128-bit reads is conflict-free.
__device__ __forceinline__ int q4k_act_slot(int piece16) {  // index of a 16-byte piece -> byte offset
    const int g = piece16 >> 2, j = piece16 & 3;
    return (((g >> 5) * 4 + j) << 9) + ((g & 31) << 4);
}

// ---------------------------------------------------------------- per-row dot products from shared memory
// Four lanes share a super-block: lane c of them owns the 32 nibble bytes of sub-blocks 2c (low
// nibbles) and 2c+1 (high nibbles), so the 6-bit scale decode is paid once per 64 weights. The
// high nibbles are used in place (16 x their value, as unsigned bytes); the factor leaves as an
// exact shift of the integer sum.
template <int NC>
__device__ __forceinline__ void row_q4_K(const uint8_t *row, int nsb, const uint8_t *sact, int act_stride,
                                         const float *ad, const int16_t *ab, int lane, int part, int wpr, float (&f)[NC]) {
    const int c = lane & 3;
    const int sh = (c & 1) * 16;
    for (int it = part; it * 8 < nsb; it += wpr) {
        const int sb = it * 8 + (lane >> 2);
        if (sb >= nsb) break;
        const uint8_t *blk = row + sb * 144;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * c);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * c);
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        // 6-bit scales/mins of sub-blocks 2c and 2c+1 (get_scale_min_k4, ggml-quants.c:880-887)
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
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint8_t *a = sact + it * 2048 + lane * 16;
#pragma unroll
        for (int n = 0; n < NC; n++) {
            const int4 a0 = *reinterpret_cast<const int4 *>(a + n * act_stride);
            const int4 a1 = *reinterpret_cast<const int4 *>(a + n * act_stride + 512);
            const int4 a2 = *reinterpret_cast<const int4 *>(a + n * act_stride + 1024);
            const int4 a3 = *reinterpret_cast<const int4 *>(a + n * act_stride + 1536);
            int il = __dp4a((int)(w[0] & 0x0f0f0f0fu), a0.x, 0), il2 = __dp4a((int)(w[4] & 0x0f0f0f0fu), a1.x, 0);
            il = __dp4a((int)(w[1] & 0x0f0f0f0fu), a0.y, il);
            il2 = __dp4a((int)(w[5] & 0x0f0f0f0fu), a1.y, il2);
            il = __dp4a((int)(w[2] & 0x0f0f0f0fu), a0.z, il);
            il2 = __dp4a((int)(w[6] & 0x0f0f0f0fu), a1.z, il2);
            il = __dp4a((int)(w[3] & 0x0f0f0f0fu), a0.w, il);
            il2 = __dp4a((int)(w[7] & 0x0f0f0f0fu), a1.w, il2);
            int ih = dp4a_us(w[0] & 0xf0f0f0f0u, a2.x, 0), ih2 = dp4a_us(w[4] & 0xf0f0f0f0u, a3.x, 0);
            ih = dp4a_us(w[1] & 0xf0f0f0f0u, a2.y, ih);
            ih2 = dp4a_us(w[5] & 0xf0f0f0f0u, a3.y, ih2);
            ih = dp4a_us(w[2] & 0xf0f0f0f0u, a2.z, ih);
            ih2 = dp4a_us(w[6] & 0xf0f0f0f0u, a3.z, ih2);
            ih = dp4a_us(w[3] & 0xf0f0f0f0u, a2.w, ih);
            ih2 = dp4a_us(w[7] & 0xf0f0f0f0u, a3.w, ih2);
            // bsums of the four 16-value groups of this chunk: two per sub-block
            const int2 bs = *reinterpret_cast<const int2 *>(ab + n * (nsb * 16) + sb * 16 + 4 * c);
            const int b_lo = (int)(short)(bs.x & 0xffff) + (bs.x >> 16), b_hi = (int)(short)(bs.y & 0xffff) + (bs.y >> 16);
            const int acc = sc_lo * (il + il2) + sc_hi * ((ih + ih2) >> 4);
            const int macc = m_lo * b_lo + m_hi * b_hi;
            const float yd = ad[n * nsb + sb];
            f[n] += yd * (dm.x * (float)acc - dm.y * (float)macc);
        }
    }
}

// 34-byte / 18-byte blocks are only 2-byte aligned: read whole words and realign by 16 bits.
template <int NC>
__device__ __forceinline__ void row_q8_0(const uint8_t *row, int K, const int8_t *aq, const float *ad, int lane,
                                         int part, int wpr, float (&f)[NC]) {
    const int nblk = K / 32;
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
            const int4 *a = reinterpret_cast<const int4 *>(aq + n * K + b * 32);
            const int4 a0 = a[0], a1 = a[1];
            int s = __dp4a((int)qs[0], a0.x, 0);
            s = __dp4a((int)qs[1], a0.y, s);
            s = __dp4a((int)qs[2], a0.z, s);
            s = __dp4a((int)qs[3], a0.w, s);
            s = __dp4a((int)qs[4], a1.x, s);
            s = __dp4a((int)qs[5], a1.y, s);
            s = __dp4a((int)qs[6], a1.z, s);
            s = __dp4a((int)qs[7], a1.w, s);
            f[n] += (float)s * (d * ad[n * nblk + b]);
        }
    }
}

template <int NC>
__device__ __forceinline__ void row_q4_0(const uint8_t *row, int K, const int8_t *aq, const float *ad, int lane,
                                         int part, int wpr, float (&f)[NC]) {
    const int nblk = K / 32;
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
            const int4 *a = reinterpret_cast<const int4 *>(aq + n * K + b * 32);
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
            f[n] += (float)s * d * ad[n * nblk + b];
        }
    }
}

// ---------------------------------------------------------------- the streaming kernel
// One CTA per SM. Warp GEMV_CW (lane 0) is the producer: it refills a stage as soon as every
// consumer warp has released it (empty barrier, one arrival per warp). The 16 consumer warps never
// meet at a CTA-wide barrier: each waits for a stage, reduces its own rows and releases it.
template <int TYPE, int NC>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
k_gemv_stream(const uint8_t *__restrict__ W, int row_bytes, int64_t M, int K, const int8_t *__restrict__ aq,
              const float *__restrict__ ad, const int16_t *__restrict__ ab, float *__restrict__ y, int64_t ldy, int n0,
              int rows_per_tile, int wpr_log, int stage_stride, int act_stride, int *__restrict__ err) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full[GEMV_STAGES], empty[GEMV_STAGES];
    __shared__ float partial[2][GEMV_CW][NC];
    // The weights do not depend on the kernel before this one: the producer streams them without waiting for it.
    // The consumers wait before they touch the activations or write a result.
    griddep_launch();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wpr = 1 << wpr_log;
    const int rows_per_pass = GEMV_CW >> wpr_log;
    const int64_t n_tiles = (M + rows_per_tile - 1) / rows_per_tile;
    const int my_tiles = blockIdx.x < n_tiles ? (int)((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    uint8_t *sact = smem + GEMV_STAGES * stage_stride;
    if (tid == 0) {
        for (int s = 0; s < GEMV_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == GEMV_CW) {
        if (lane != 0) return;
        int issued = 0;
        bool ok = true;
        for (int i = 0; i < my_tiles && ok; i++) {
            const int s = i & (GEMV_STAGES - 1);
            if (i >= GEMV_STAGES) ok = mbar_wait(&empty[s], (uint32_t)(((i / GEMV_STAGES) - 1) & 1));
            if (!ok) break;
            const int64_t r0 = (blockIdx.x + (int64_t)i * gridDim.x) * rows_per_tile;
            const int rows = (int)min((int64_t)rows_per_tile, M - r0);
            const uint32_t bytes = (uint32_t)(rows * row_bytes);
            mbar_expect_tx(&full[s], bytes);
            bulk_g2s(smem + s * stage_stride, W + r0 * row_bytes, bytes, &full[s]);
            issued = i + 1;
        }
        if (!ok) {
            // the consumers stopped releasing stages: record it, then wait (bounded) for the copies
            // still in flight before the CTA's shared memory is released
            atomicExch(err, 1);
            for (int j = max(0, issued - GEMV_STAGES); j < issued; j++)
                mbar_wait(&full[j & (GEMV_STAGES - 1)], (uint32_t)((j / GEMV_STAGES) & 1));
        }
        return;
    }

    // ---- consumers
    griddep_wait();
    aq += (int64_t)n0 * K;
    if (TYPE == TLB_TYPE_Q4_K) {
        // int8 codes of this pass's columns -> shared memory, in the lane order of row_q4_K
        const int pieces = K / 16;
        for (int n = 0; n < NC; n++)
            for (int p = tid; p < pieces; p += GEMV_CW * 32)
                *reinterpret_cast<int4 *>(sact + n * act_stride + q4k_act_slot(p)) =
                    *reinterpret_cast<const int4 *>(aq + (int64_t)n * K + p * 16);
        named_bar_sync(1, GEMV_CW * 32);
    }
    const int nblk = TYPE == TLB_TYPE_Q4_K ? K / 256 : K / 32;
    ad += (int64_t)n0 * nblk;
    if (TYPE == TLB_TYPE_Q4_K) ab += (int64_t)n0 * (K / 16);
    y += (int64_t)n0 * ldy;
    const int grp = warp >> wpr_log, part = warp & (wpr - 1);
    int pbuf = 0;
    for (int i = 0; i < my_tiles; i++) {
        const int s = i & (GEMV_STAGES - 1);
        if (!mbar_wait(&full[s], (uint32_t)((i / GEMV_STAGES) & 1))) {
            if (lane == 0) atomicExch(err, 1);
            break;  // this warp stops releasing stages; the producer's bounded wait ends the CTA
        }
        const int64_t r0 = (blockIdx.x + (int64_t)i * gridDim.x) * rows_per_tile;
        const int rows = (int)min((int64_t)rows_per_tile, M - r0);
        const uint8_t *base = smem + s * stage_stride;
        for (int r = grp; r < rows; r += rows_per_pass) {
            float f[NC];
#pragma unroll
            for (int n = 0; n < NC; n++) f[n] = 0.f;
            const uint8_t *row = base + r * row_bytes;
            if (TYPE == TLB_TYPE_Q4_K) row_q4_K<NC>(row, nblk, sact, act_stride, ad, ab, lane, part, wpr, f);
            else if (TYPE == TLB_TYPE_Q8_0) row_q8_0<NC>(row, K, aq, ad, lane, part, wpr, f);
            else row_q4_0<NC>(row, K, aq, ad, lane, part, wpr, f);
#pragma unroll
            for (int n = 0; n < NC; n++) f[n] = warp_sum(f[n]);
            if (wpr == 1) {
                if (lane == 0) {
#pragma unroll
                    for (int n = 0; n < NC; n++) y[n * ldy + r0 + r] = f[n];
                }
            } else {
                // the warps of a row combine their partial sums in a fixed order; the pair of
                // buffers lets the fastest warp run one row ahead of the one that adds them up
                if (lane == 0) {
#pragma unroll
                    for (int n = 0; n < NC; n++) partial[pbuf][warp][n] = f[n];
                }
                named_bar_sync(2 + grp, 32 * wpr);
                if (part == 0 && lane < NC) {
                    float v = 0.f;
                    for (int pp = 0; pp < wpr; pp++) v += partial[pbuf][warp + pp][lane];
                    y[lane * ldy + r0 + r] = v;
                }
                pbuf ^= 1;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
}

static uint64_t q4k_act_bytes(int64_t K) { return (uint64_t)((K / 256 + 7) / 8) * 2048; }

bool gemv_supported(uint32_t type, int64_t K, int64_t M, int64_t N) {
    if (type != TLB_TYPE_Q4_K && type != TLB_TYPE_Q8_0 && type != TLB_TYPE_Q4_0) return false;
    if (K % 256 != 0 || M < 1 || N < 1 || K > (1 << 20)) return false;
    if (type == TLB_TYPE_Q4_K && q4k_act_bytes(K) > GEMV_ACT_SMEM) return false;
    const int64_t rb = (int64_t)tlb_row_size(type, K);
    return rb % 16 == 0 && rb + GEMV_PAD <= GEMV_STAGE_BYTES;
}

template <int TYPE, int NC>
static void set_attr() {
    cudaFuncSetAttribute(k_gemv_stream<TYPE, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         GEMV_STAGES * (GEMV_STAGE_BYTES + 128) + (TYPE == TLB_TYPE_Q4_K ? GEMV_ACT_SMEM : 0));
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
    int max_rows = (int)((GEMV_STAGE_BYTES - GEMV_PAD) / rb);
    // keep every SM busy: no more rows per tile than gives each SM a few tiles
    const int64_t want_tiles = (int64_t)sm_count * 4;
    const int64_t cap = (M + want_tiles - 1) / want_tiles;
    if (max_rows > cap) max_rows = (int)(cap < 1 ? 1 : cap);
    const int64_t units = TYPE == TLB_TYPE_Q4_K ? (K / 256 + 7) / 8 : (K / 32 + 31) / 32;  // loop trips of one warp
    // rows per tile: a whole number of rows per consumer warp, or (fewer rows than warps) the
    // count that keeps most warps busy when 2^j warps share a row
    int rows_per_tile = max_rows, wpr_log = 0;
    if (max_rows >= GEMV_CW) {
        rows_per_tile = max_rows / GEMV_CW * GEMV_CW;
    } else {
        int best = -1;
        for (int r = 1; r <= max_rows; r++) {
            int wl = 0;
            while ((2 << wl) * r <= GEMV_CW && (2 << wl) <= units) wl++;
            const int used = r << wl;
            if (used >= best) { best = used; rows_per_tile = r; wpr_log = wl; }
        }
    }
    const int stage_stride = (int)(((int64_t)rows_per_tile * rb + GEMV_PAD + 127) / 128 * 128);
    const int64_t n_tiles = (M + rows_per_tile - 1) / rows_per_tile;
    const int grid = (int)(n_tiles < sm_count ? n_tiles : sm_count);
    const int act_stride = TYPE == TLB_TYPE_Q4_K ? (int)q4k_act_bytes(K) : 0;
    const int nc_max = TYPE == TLB_TYPE_Q4_K ? (int)std::min<int64_t>(4, GEMV_ACT_SMEM / act_stride) : 4;
    const char *ab = (const char *)act;
    const int8_t *aq = (const int8_t *)(ab + a.qs_off);
    const float *ad = (const float *)(ab + a.d_off);
    const int16_t *bs = (const int16_t *)(ab + a.bsum_off);
    cudaError_t e = cudaSuccess;
    for (int n0 = 0; n0 < a.N && e == cudaSuccess;) {
        const int nc = (int)std::min<int64_t>(nc_max, a.N - n0);
        const size_t smem = (size_t)GEMV_STAGES * stage_stride + (size_t)nc * act_stride;
#define GO(NCV)                                                                                                        \
    e = launch_pdl(k_gemv_stream<TYPE, NCV>, dim3((unsigned)grid), dim3(GEMV_THREADS), smem, st, (const uint8_t *)W, (int)rb, M, (int)K, aq, ad, bs, \
                   y, ldy, n0, rows_per_tile, wpr_log, stage_stride, act_stride, err)
        switch (nc) {
            case 1: GO(1); break;
            case 2: GO(2); break;
            case 3: GO(3); break;
            default: GO(4); break;
        }
#undef GO
        n0 += nc;
    }
    return e;
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
    } else if (p.wtype != TLB_TYPE_Q8_0 && p.wtype != TLB_TYPE_Q4_0 && p.wtype != TLB_TYPE_Q4_K) {
        // the other block types: decoded weights times the f32 activations, the reference executor's own arithmetic
        // for every type (crates/kernels/src/cuda/native/mm.cu:16-42)
        const uint8_t *xcol = X + n * p.x.nb[1] + i2 * p.x.nb[2] + i3 * p.x.nb[3];
        for (int64_t k = lane; k < K; k += 32) f += dq_elem(wrow, p.wtype, k) * *reinterpret_cast<const float *>(xcol + k * p.x.nb[0]);
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
