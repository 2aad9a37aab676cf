// FLASH_ATTN_EXT for prompt-sized query counts on the 5th-generation tensor cores (head size 128, f16 keys and values,
// optional f16 mask, no soft cap, no ALiBi; everything else takes k_flash.cu). Same arithmetic as k_flash.cu:
// softmax(scale * f16(Q) K^T + mask) V with f16 operands, f32 scores, f32 running sums, P rounded to f16.
//
// Three launches per node:
//   1. k_fa_pack_*: Q (f32 -> f16), K and V^T go into 32 KB blobs of 128 rows x 128 columns in the K-major core-matrix
//      layout that tcgen05.mma reads from shared memory ([row / 8][16 chunks of 8 elements][row % 8][16 bytes]),
//      so that the main kernel moves whole tiles with one bulk copy each and needs no transposition.
//   2. k_fa_tile_flags: one byte per (query tile, key tile) of the mask: all -inf (the tile is skipped, the upper
//      triangle of a causal mask), all zero (no mask values are read), or mixed.
//   3. k_fa_tc: a CTA owns 128 queries of one (head, batch). Tensor memory holds two score accumulators S (128 columns
//      each), the output accumulator O (128 columns) and two P operands (f16, 64 columns each). One warp copies tiles,
//      one issues MMAs (S = Q K^T: 8 x 128x128x16 from shared memory; O += P V: 8 x 128x128x16 with P read from tensor
//      memory), eight warps do the softmax, two threads per query row with 64 score columns each: they pull their half
//      of the row out of tensor memory, agree on the row's maximum through shared memory, take exp2 and their part of
//      the sum, and put P back (one thread per row spent 3500-4000 cycles per key tile on its own serial instruction
//      stream and the tensor-memory round trips; splitting the row halves that). S is double buffered, so the tensor core works on the next tile's
//      scores while the exponentials of this one are taken. The running maximum that the exponents refer to is only
//      moved when a row's maximum has grown by more than 2^8 (the factor cancels in the final division; P stays far
//      inside the f16 range), so O in tensor memory is rescaled rarely instead of once per tile.
// Every wait is bounded (tc_common.cuh); a wait that gives up sets the program's error word.
#include <cuda.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kernels.h"
#include "pdl.cuh"
#include "tc_common.cuh"

namespace tlb {

namespace fat {
constexpr int T = 128;                    // queries per CTA, keys per tile, head size
constexpr int TILE_BYTES = T * T * 2;     // 32 KB
constexpr int THREADS = 384;              // warp 0 copies, warp 1 issues MMAs, warps 2-3 idle, warps 4-11 softmax
constexpr int SM_WARP0 = 4, SM_WARPS = 8; // two threads per query row: warps 4-7 take score columns 0-63, warps 8-11 columns 64-127
constexpr uint32_t S_COL0 = 0, O_COL0 = 256, P_COL0 = 384;
constexpr float RESCALE_STEP = 8.f;       // in the base-2 domain

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// byte offset of (row, 16-byte chunk c of the row) inside a 128 x 128 f16 blob
__device__ __forceinline__ int blob_off(int row, int c) { return (row >> 3) * 2048 + c * 128 + (row & 7) * 16; }
}  // namespace fat

// ---------------------------------------------------------------- operand packing
// grid (query tile, head, batch): q f32 [D, nq, nh, nb] (strided) -> f16 blob; rows past nq are zero
__global__ void __launch_bounds__(256) k_fa_pack_q(FlashArgs p, const uint8_t *__restrict__ q, uint8_t *__restrict__ out, int n_qt) {
    griddep_launch();
    griddep_wait();
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    uint8_t *o = out + (((size_t)b * p.nh + h) * n_qt + qt) * fat::TILE_BYTES;
    const uint8_t *qb = q + (int64_t)h * p.q.nb[2] + (int64_t)b * p.q.nb[3];
    for (int u = threadIdx.x; u < fat::T * 16; u += blockDim.x) {
        const int row = u >> 4, c = u & 15, qr = qt * fat::T + row;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (qr < p.nq) {
            const float *src = reinterpret_cast<const float *>(qb + (int64_t)qr * p.q.nb[1]) + c * 8;
            const float4 a = *reinterpret_cast<const float4 *>(src), d = *reinterpret_cast<const float4 *>(src + 4);
            v = make_uint4(fat::pack_h2(a.x, a.y), fat::pack_h2(a.z, a.w), fat::pack_h2(d.x, d.y), fat::pack_h2(d.z, d.w));
        }
        *reinterpret_cast<uint4 *>(o + fat::blob_off(row, c)) = v;
    }
}
// grid (key tile, kv head, batch): k f16 [D, nkv, nhkv, nb] -> blob (rows = keys); v -> blob of V^T (rows = head
// dimensions, columns = keys). Keys past nkv are zero.
__global__ void __launch_bounds__(256) k_fa_pack_kv(FlashArgs p, const uint8_t *__restrict__ k, const uint8_t *__restrict__ v,
                                                     uint8_t *__restrict__ kout, uint8_t *__restrict__ vout, int n_kt) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) __half vs[fat::T][fat::T + 8];
    const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const size_t tile = (((size_t)b * p.nhkv + hk) * n_kt + kt) * fat::TILE_BYTES;
    const uint8_t *kb = k + (int64_t)hk * p.k.nb[2] + (int64_t)b * p.k.nb[3];
    const uint8_t *vb = v + (int64_t)hk * p.v.nb[2] + (int64_t)b * p.v.nb[3];
    for (int u = threadIdx.x; u < fat::T * 16; u += blockDim.x) {
        const int row = u >> 4, c = u & 15, key = kt * fat::T + row;
        uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (key < p.nkv) {
            kv = *reinterpret_cast<const uint4 *>(kb + (int64_t)key * p.k.nb[1] + c * 16);
            vv = *reinterpret_cast<const uint4 *>(vb + (int64_t)key * p.v.nb[1] + c * 16);
        }
        *reinterpret_cast<uint4 *>(kout + tile + fat::blob_off(row, c)) = kv;
        *reinterpret_cast<uint4 *>(&vs[row][c * 8]) = vv;
    }
    __syncthreads();
    for (int u = threadIdx.x; u < fat::T * 16; u += blockDim.x) {
        const int d = u & 127, kc = u >> 7;   // consecutive threads take consecutive head dimensions of the same 8 keys
        __half h[8];
#pragma unroll
        for (int e = 0; e < 8; e++) h[e] = vs[kc * 8 + e][d];
        *reinterpret_cast<uint4 *>(vout + tile + fat::blob_off(d, kc)) = *reinterpret_cast<const uint4 *>(h);
    }
}
// grid (key tile, query tile, mask plane): 0 = every mask value of the tile is -inf, 1 = every one is zero, 2 = mixed
__global__ void __launch_bounds__(256) k_fa_tile_flags(FlashArgs p, const uint8_t *__restrict__ mask, uint8_t *__restrict__ flags, int n_qt, int n_kt) {
    griddep_launch();
    griddep_wait();
    const int kt = blockIdx.x, qt = blockIdx.y, plane = blockIdx.z;
    const int m2 = plane % p.m_ne2, m3 = plane / p.m_ne2;
    const uint8_t *mb = mask + (int64_t)m2 * p.m.nb[2] + (int64_t)m3 * p.m.nb[3];
    bool not_dead = false, not_plain = false;
    for (int u = threadIdx.x; u < fat::T * fat::T; u += blockDim.x) {
        const int row = u >> 7, col = u & 127, qr = qt * fat::T + row, key = kt * fat::T + col;
        if (qr < p.nq && key < p.nkv) {
            const unsigned short bits = __half_as_ushort(reinterpret_cast<const __half *>(mb + (int64_t)qr * p.m.nb[1])[key]);
            not_dead |= bits != 0xfc00;
            not_plain |= (bits & 0x7fff) != 0;
        }
    }
    const int nd = __syncthreads_or(not_dead), np = __syncthreads_or(not_plain);
    if (threadIdx.x == 0) flags[((size_t)plane * n_qt + qt) * n_kt + kt] = !nd ? 0 : (np ? 2 : 1);
}

// ---------------------------------------------------------------- the attention kernel
struct FaTcParams {
    const uint8_t *qp, *kp, *vt, *flags, *mask;   // flags and mask null without a mask
    TView m;
    int m_ne2, m_ne3;
    float *out;
    int nq, nkv, nh, nhkv, nb, n_qt, n_kt;
    float scale_log2, log2e;
    int *err;
};

__global__ void __launch_bounds__(fat::THREADS, 1) k_fa_tc(FaTcParams p) {
    using namespace tc;
    constexpr int T = fat::T;
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(T >> 3) << 17) | ((uint32_t)(T >> 4) << 24);   // f16 x f16 -> f32, K-major A and B
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (su32(smem_raw) & 1023u)) & 1023u);
    uint8_t *qs = smem, *ks = qs + fat::TILE_BYTES, *vs = ks + 2 * fat::TILE_BYTES;
    __shared__ uint64_t bar_q, bar_k[2], bar_v[2], bar_kfree[2], bar_vfree[2], bar_s[2], bar_sfree[2], bar_p[2], bar_pv;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_fail, n_live_s;
    __shared__ float pair_x[2][fat::T];   // what the two threads of a row tell each other: the maximum of their half, at the end their sum
    __shared__ uint16_t live_kt[512];   // key tiles that are not skipped, with their flag in the top bits
    volatile int *fail = &s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = p.n_qt - 1 - (int)blockIdx.x;   // the longest rows of a causal mask first
    const int h = blockIdx.y, b = blockIdx.z, hk = h / (p.nh / p.nhkv);
    griddep_launch();
    if (tid == 0) {
        mbar_init(&bar_q, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&bar_k[i], 1);
            mbar_init(&bar_v[i], 1);
            mbar_init(&bar_kfree[i], 1);
            mbar_init(&bar_vfree[i], 1);
            mbar_init(&bar_s[i], 1);
            mbar_init(&bar_sfree[i], fat::SM_WARPS);
            mbar_init(&bar_p[i], fat::SM_WARPS);
        }
        mbar_init(&bar_pv, 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&tmem_base_s, 512);
    if (warp == 2) {
        // the key tiles this CTA visits (the flags were written by the launch in front)
        griddep_wait();
        if (lane == 0) {
            const uint8_t *fl = p.flags ? p.flags + ((size_t)((b % p.m_ne3) * p.m_ne2 + (h % p.m_ne2)) * p.n_qt + qt) * p.n_kt : nullptr;
            int n = 0;
            for (int kt = 0; kt < p.n_kt; kt++) {
                int f = fl ? fl[kt] : 1;
                if (f == 0) continue;
                if (kt == p.n_kt - 1 && (p.nkv & (T - 1))) f |= 4;   // keys past the last one are masked by index
                live_kt[n++] = (uint16_t)(kt | (f << 12));
            }
            n_live_s = n;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    const int n_live = n_live_s;

    if (warp == 0) {
        // ---- tile copies
        if (lane == 0 && n_live > 0) {
            griddep_wait();
            mbar_expect_tx(&bar_q, fat::TILE_BYTES);
            bulk_g2s(qs, p.qp + (((size_t)b * p.nh + h) * p.n_qt + qt) * fat::TILE_BYTES, fat::TILE_BYTES, &bar_q);
            const size_t kv0 = ((size_t)b * p.nhkv + hk) * p.n_kt;
            for (int j = 0; j < n_live; j++) {
                const int s = j & 1, kt = live_kt[j] & 0xfff;
                if (j >= 2) mbar_wait_nap(&bar_kfree[s], ((j >> 1) - 1) & 1, fail, 32);
                mbar_expect_tx(&bar_k[s], fat::TILE_BYTES);
                bulk_g2s(ks + s * fat::TILE_BYTES, p.kp + (kv0 + kt) * fat::TILE_BYTES, fat::TILE_BYTES, &bar_k[s]);
                if (j >= 2) mbar_wait_nap(&bar_vfree[s], ((j >> 1) - 1) & 1, fail, 32);
                mbar_expect_tx(&bar_v[s], fat::TILE_BYTES);
                bulk_g2s(vs + s * fat::TILE_BYTES, p.vt + (kv0 + kt) * fat::TILE_BYTES, fat::TILE_BYTES, &bar_v[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the whole warp runs the loop (converged), one elected lane issues
        const bool leader = elect_one();
        if (n_live > 0) {
            const uint64_t q_desc = smem_desc(su32(qs), 128, 2048);
            auto issue_qk = [&](int j) {
                const int s = j & 1;
                mbar_wait_nap(&bar_k[s], (j >> 1) & 1, fail, 32);
                if (j >= 2) mbar_wait_nap(&bar_sfree[s], ((j >> 1) - 1) & 1, fail, 32);   // S[s] has been read by the softmax warps
                tc_fence_after();
                if (leader) {
                    const uint64_t k_desc = smem_desc(su32(ks + s * fat::TILE_BYTES), 128, 2048);
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        umma_f16(tmem_base + fat::S_COL0 + (uint32_t)(s * T), q_desc + (uint64_t)(k * 16), k_desc + (uint64_t)(k * 16), IDESC, k ? 1u : 0u);
                    umma_commit(&bar_s[s]);
                    umma_commit(&bar_kfree[s]);
                }
                __syncwarp();
            };
            mbar_wait_nap(&bar_q, 0, fail, 32);
            issue_qk(0);
            for (int j = 0; j < n_live; j++) {
                const int s = j & 1;
                if (j + 1 < n_live) issue_qk(j + 1);
                mbar_wait_nap(&bar_p[s], (j >> 1) & 1, fail, 32);
                mbar_wait_nap(&bar_v[s], (j >> 1) & 1, fail, 32);
                tc_fence_after();
                if (leader) {
                    const uint64_t v_desc = smem_desc(su32(vs + s * fat::TILE_BYTES), 128, 2048);
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        umma_f16_ta(tmem_base + fat::O_COL0, tmem_base + fat::P_COL0 + (uint32_t)(s * 64 + k * 8), v_desc + (uint64_t)(k * 16), IDESC,
                                    (j | k) ? 1u : 0u);
                    umma_commit(&bar_pv);
                    umma_commit(&bar_vfree[s]);
                }
                __syncwarp();
            }
        }
    } else if (warp >= fat::SM_WARP0) {
        // ---- softmax: two threads per query row (64 score columns each); the pair shares a lane quadrant and meets at
        // a named barrier of its own (64 threads) to agree on the row's maximum
        const int quad = warp & 3, half = (warp - fat::SM_WARP0) >> 2;
        const int row = quad * 32 + lane, qr = qt * T + row;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };
        const __half *mrow = nullptr;
        if (p.mask)
            mrow = reinterpret_cast<const __half *>(p.mask + (int64_t)(h % p.m_ne2) * p.m.nb[2] + (int64_t)(b % p.m_ne3) * p.m.nb[3] +
                                                    (int64_t)min(qr, p.nq - 1) * p.m.nb[1]);
        float m_ref = 0.f, l = 0.f;
        bool have_ref = false;   // m_ref is the maximum the exponents refer to; unset until the row has seen a finite score
        for (int j = 0; j < n_live; j++) {
            const int s = j & 1, kt = live_kt[j] & 0xfff, flag = live_kt[j] >> 12;
            const int key0 = kt * T + half * 64;
            mbar_wait_nap(&bar_s[s], (j >> 1) & 1, fail, 0);
            tc_fence_after();
            float x[64];
            fat::tmem_ld32(lane_base + fat::S_COL0 + (uint32_t)(s * T + half * 64), reinterpret_cast<uint32_t *>(x));
            fat::tmem_ld32(lane_base + fat::S_COL0 + (uint32_t)(s * T + half * 64 + 32), reinterpret_cast<uint32_t *>(x) + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_sfree[s]);
            // scores in the base-2 domain
#pragma unroll
            for (int i = 0; i < 64; i++) x[i] *= p.scale_log2;
            if (flag & 2) {
                const bool full = key0 + 64 <= p.nkv;
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (full) {
                        v = *reinterpret_cast<const uint4 *>(mrow + key0 + c * 8);
                    } else {
                        __half t[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) t[e] = key0 + c * 8 + e < p.nkv ? mrow[key0 + c * 8 + e] : __ushort_as_half(0);
                        v = *reinterpret_cast<const uint4 *>(t);
                    }
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(h2[e]);
                        x[c * 8 + 2 * e] += f.x * p.log2e;
                        x[c * 8 + 2 * e + 1] += f.y * p.log2e;
                    }
                }
            }
            if (flag & 4) {
#pragma unroll
                for (int i = 0; i < 64; i++)
                    if (key0 + i >= p.nkv) x[i] = -CUDART_INF_F;
            }
            float mx = x[0];
#pragma unroll
            for (int i = 1; i < 64; i++) mx = fmaxf(mx, x[i]);
            pair_x[half][row] = mx;
            pair_sync();
            mx = fmaxf(mx, pair_x[half ^ 1][row]);
            pair_sync();   // both have read before either writes the next tile's value
            // the reference maximum moves only when this row's maximum has outgrown it by more than the step (the two
            // threads of a row see the same numbers and take the same decisions)
            float alpha = 1.f;
            if (!have_ref) {
                if (mx != -CUDART_INF_F) {
                    m_ref = mx;
                    have_ref = true;   // nothing has been accumulated for this row yet: O and l are zero
                }
            } else if (mx > m_ref + fat::RESCALE_STEP) {
                alpha = fat::ex2(m_ref - mx);
                m_ref = mx;
            }
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
                // O of the tiles before has to be complete before it is scaled (j > 0 here: alpha is 1 on the first tile);
                // each thread scales its half of the row's output columns
                mbar_wait_nap(&bar_pv, (j - 1) & 1, fail, 0);
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 2; c++) {
                    uint32_t o[32];
                    fat::tmem_ld32(lane_base + fat::O_COL0 + (uint32_t)(half * 64 + c * 32), o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    fat::tmem_st32(lane_base + fat::O_COL0 + (uint32_t)(half * 64 + c * 32), o);
                }
                tmem_st_wait();
                l *= alpha;
            }
            // P = exp2(x - m_ref) as f16 pairs; this thread's part of the row sum in f32
            uint32_t pk[32];
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const float e0 = fat::ex2(x[i] - m_ref), e1 = fat::ex2(x[i + 1] - m_ref);
                sum += e0 + e1;
                pk[i / 2] = fat::pack_h2(e0, e1);
            }
            l += sum;
            fat::tmem_st32(lane_base + fat::P_COL0 + (uint32_t)(s * 64 + half * 32), pk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_p[s]);
        }
        // ---- O / l -> out [D, nh, nq, nb]: the row sum is the two threads' parts together, each writes its 64 columns
        pair_x[half][row] = l;
        pair_sync();
        l += pair_x[half ^ 1][row];
        if (n_live > 0) {
            mbar_wait_nap(&bar_pv, (n_live - 1) & 1, fail, 0);
            tc_fence_after();
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        float *dst = p.out + (((int64_t)b * p.nq + qr) * p.nh + h) * T + half * 64;
#pragma unroll 1
        for (int c = 0; c < 2; c++) {
            uint32_t o[32];
            if (n_live > 0) {
                fat::tmem_ld32(lane_base + fat::O_COL0 + (uint32_t)(half * 64 + c * 32), o);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = 0u;
            }
            if (qr < p.nq) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4 *>(dst + c * 32 + i) = make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                                                                __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && s_fail && p.err) atomicExch(p.err, 2);
}

// ---------------------------------------------------------------- host side
static size_t fa_tc_smem() { return 5 * (size_t)fat::TILE_BYTES + 1024; }
void flash_tc_configure() { cudaFuncSetAttribute(k_fa_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_tc_smem()); }

bool flash_tc_supported(const FlashArgs &p, bool has_mask) {
    if (getenv("TLB_NO_FLASH_TC") || !tc_available()) return false;
    if (p.d != fat::T || p.dv != fat::T || p.k_ty != TLB_TYPE_F16 || p.v_ty != TLB_TYPE_F16 || p.softcap != 0.f || p.max_bias != 0.f) return false;
    if (p.nq < 64 || p.nkv < 1 || (p.nkv + fat::T - 1) / fat::T > 512 || p.nh % p.nhkv != 0) return false;
    if (p.q.nb[1] % 16 || p.q.nb[2] % 16 || p.q.nb[3] % 16) return false;
    if (has_mask && (p.m.nb[1] % 16 || p.m.nb[2] % 16 || p.m.nb[3] % 16)) return false;
    return true;
}

struct FaTcLayout {
    int n_qt, n_kt;
    uint64_t q_off, k_off, v_off, f_off, bytes;
};
static FaTcLayout fa_tc_layout(const FlashArgs &p, bool has_mask) {
    FaTcLayout L;
    L.n_qt = (p.nq + fat::T - 1) / fat::T;
    L.n_kt = (p.nkv + fat::T - 1) / fat::T;
    L.q_off = 0;
    L.k_off = L.q_off + (uint64_t)p.nb * p.nh * L.n_qt * fat::TILE_BYTES;
    L.v_off = L.k_off + (uint64_t)p.nb * p.nhkv * L.n_kt * fat::TILE_BYTES;
    L.f_off = L.v_off + (uint64_t)p.nb * p.nhkv * L.n_kt * fat::TILE_BYTES;
    L.bytes = L.f_off + (has_mask ? ((uint64_t)p.m_ne2 * p.m_ne3 * L.n_qt * L.n_kt + 255) / 256 * 256 : 0);
    return L;
}
uint64_t flash_tc_scratch_bytes(const FlashArgs &p, bool has_mask) { return fa_tc_layout(p, has_mask).bytes; }

cudaError_t launch_flash_attn_tc(const FlashArgs &p, const void *q, const void *k, const void *v, const void *mask, float *out, void *scratch,
                                 int *err, cudaStream_t st) {
    if (p.nq == 0 || p.nh == 0 || p.nb == 0) return cudaSuccess;
    const FaTcLayout L = fa_tc_layout(p, mask != nullptr);
    uint8_t *sc = (uint8_t *)scratch;
    cudaError_t e = launch_pdl(k_fa_pack_q, dim3((unsigned)L.n_qt, (unsigned)p.nh, (unsigned)p.nb), dim3(256), 0, st, p, (const uint8_t *)q, sc + L.q_off, L.n_qt);
    if (e != cudaSuccess) return e;
    e = launch_pdl(k_fa_pack_kv, dim3((unsigned)L.n_kt, (unsigned)p.nhkv, (unsigned)p.nb), dim3(256), 0, st, p, (const uint8_t *)k, (const uint8_t *)v,
                   sc + L.k_off, sc + L.v_off, L.n_kt);
    if (e != cudaSuccess) return e;
    if (mask) {
        e = launch_pdl(k_fa_tile_flags, dim3((unsigned)L.n_kt, (unsigned)L.n_qt, (unsigned)(p.m_ne2 * p.m_ne3)), dim3(256), 0, st, p, (const uint8_t *)mask,
                       sc + L.f_off, L.n_qt, L.n_kt);
        if (e != cudaSuccess) return e;
    }
    FaTcParams a{};
    a.qp = sc + L.q_off;
    a.kp = sc + L.k_off;
    a.vt = sc + L.v_off;
    a.flags = mask ? sc + L.f_off : nullptr;
    a.mask = (const uint8_t *)mask;
    a.m = p.m;
    a.m_ne2 = p.m_ne2;
    a.m_ne3 = p.m_ne3;
    a.out = out;
    a.nq = p.nq;
    a.nkv = p.nkv;
    a.nh = p.nh;
    a.nhkv = p.nhkv;
    a.nb = p.nb;
    a.n_qt = L.n_qt;
    a.n_kt = L.n_kt;
    a.log2e = 1.4426950408889634f;
    a.scale_log2 = p.scale * a.log2e;
    a.err = err;
    return launch_pdl(k_fa_tc, dim3((unsigned)L.n_qt, (unsigned)p.nh, (unsigned)p.nb), dim3(fat::THREADS), fa_tc_smem(), st, a);
}

}  // namespace tlb
