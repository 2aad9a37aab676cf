// Batched MUL_MAT (9..64 activation columns) with Q4_K weights on the 5th-generation tensor cores.
//
// Arithmetic (same integers as the reference's ggml-cpu path, vendor/ggml/src/ggml-cpu/quants.c:696-770):
// the activations are the Q8_K codes q8 (k_quant.cu), the weights the 4-bit codes q with their 6-bit
// sub-block scales sc and mins m. Per 256-element super-block and output (row r, column c)
//     S = sum_k (sc*q)[r,k] * q8[k,c]          T = sum_j m[r,j] * bsum[j,c]
//     y += yd[c] * (d[r] * S - dmin[r] * T)
// Both sums are products of small integers: sc*q <= 945 and |q8| <= 127 are exact in f16, so
// tcgen05.mma kind::f16 with f32 accumulation in tensor memory reproduces the integer sums to 2^-24,
// and the per-sub-block scale costs nothing (it is folded into the f16 weight operand).
//
// Data movement: TMA brings a 128-row x 144-byte box of raw super-blocks (2-D tensor map over the
// weight matrix as bytes) and one packed activation blob per super-block into shared memory; all
// warps expand the nibbles into the K-major core-matrix layout (8 rows x 16 bytes, no swizzle) the
// MMA reads; one thread issues 16 MMAs (M=128, N=columns, K=16) plus one for T per super-block into a
// double-buffered TMEM accumulator; four warps drain it with tcgen05.ld and apply the f32 scales
// while the next super-block is being expanded and multiplied. K is split across CTAs; partial sums
// go to scratch and k_mmq_reduce adds them in a fixed order (deterministic).
#include <algorithm>
#include <cstdlib>
#include <cuda.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "tc_common.cuh"
#include "pdl.cuh"

namespace tlb {


// Bytes of one packed activation blob (one super-block of NPAD columns):
//   B    f16 [NPAD x 256]  core-matrix layout, sbo 4096, lbo 128       NPAD*512
//   Bmin f16 [NPAD x 16]   core-matrix layout, sbo 256,  lbo 128       NPAD*32
//   yd   f32 [NPAD]                                                    NPAD*4
static inline __host__ __device__ int tc_blob_bytes(int npad) { return (npad * 548 + 127) / 128 * 128; }

// ---------------------------------------------------------------- activation packer
// From the Q8_K activation block (qs int8 [N][K], d f32 [N][K/256], bsums int16 [N][K/16]) to the
// per-super-block blobs the MMA reads. Element order inside a 16-byte K chunk follows the order in
// which the weight nibbles come out of a 32-bit word: (0, 2, 1, 3, 4, 6, 5, 7).
__global__ void __launch_bounds__(256) k_act_pack_tc(const int8_t *__restrict__ qs, const float *__restrict__ ds,
                                                      const int16_t *__restrict__ bsums, int64_t K, int N, int npad,
                                                      uint8_t *__restrict__ out) {
    // grid (super-block, chunk of npad columns); blobs are laid out [chunk][super-block]
    const int sb = blockIdx.x;
    const int blob = tc_blob_bytes(npad);
    uint8_t *o = out + ((size_t)blockIdx.y * gridDim.x + sb) * blob;
    qs += (size_t)blockIdx.y * npad * K;
    ds += (size_t)blockIdx.y * npad * (K / 256);
    bsums += (size_t)blockIdx.y * npad * (K / 16);
    N = min(npad, N - (int)blockIdx.y * npad);
    // B tile: one 16-byte chunk per (n, kc)
    for (int u = threadIdx.x; u < npad * 32; u += blockDim.x) {
        const int n = u / 32, kc = u % 32;
        __half h[8];
        if (n < N) {
            const int8_t *src = qs + (size_t)n * K + (size_t)sb * 256 + kc * 8;
            const int perm[8] = {0, 2, 1, 3, 4, 6, 5, 7};
#pragma unroll
            for (int e = 0; e < 8; e++) h[e] = __int2half_rn((int)src[perm[e]]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++) h[e] = __float2half_rn(0.f);
        }
        *reinterpret_cast<uint4 *>(o + (size_t)(n / 8) * 4096 + kc * 128 + (n % 8) * 16) = *reinterpret_cast<const uint4 *>(h);
    }
    uint8_t *omin = o + (size_t)npad * 512;
    for (int u = threadIdx.x; u < npad * 2; u += blockDim.x) {
        const int n = u / 2, kc = u % 2;
        __half h[8];
#pragma unroll
        for (int e = 0; e < 8; e++)
            h[e] = n < N ? __int2half_rn((int)bsums[(size_t)n * (K / 16) + (size_t)sb * 16 + kc * 8 + e]) : __float2half_rn(0.f);
        *reinterpret_cast<uint4 *>(omin + (size_t)(n / 8) * 256 + kc * 128 + (n % 8) * 16) = *reinterpret_cast<const uint4 *>(h);
    }
    float *oyd = reinterpret_cast<float *>(o + (size_t)npad * 544);
    for (int n = threadIdx.x; n < npad; n += blockDim.x) oyd[n] = n < N ? ds[(size_t)n * (K / 256) + sb] : 0.f;
}

// ---------------------------------------------------------------- the GEMM
// Up to three weight matrices that share the activations (wq / wk / wv of a layer) run as one launch:
// row tiles [tile0[j], tile0[j+1]) belong to matrix j.
constexpr int TC_MAX_MATS = 3;
struct TcMaps {
    CUtensorMap m[TC_MAX_MATS];
};
struct TcParams {
    const uint8_t *act;   // packed blobs, one per super-block
    float *out[TC_MAX_MATS];   // per matrix: y (n_split == 1) or partial sums [split][N][M]
    int64_t M[TC_MAX_MATS];
    int tile0[TC_MAX_MATS + 1];
    int n_mats;
    int N, npad, nsb, sb_per_split, n_split;
    int64_t ldy;          // elements between output columns
    int *err;
    // stream-K (streamk != 0): the grid is one CTA per SM; CTA c works through the units [c T / G, (c+1) T / G) of
    // the flattened (row tile, super-block) space, T = total tiles x nsb, so every SM gets the same number of
    // super-blocks whatever the tile count. A tile that one CTA covers completely is written to y; a tile cut by
    // a CTA boundary (at most one cut per tile: the plan requires T / G >= nsb) leaves two partial results
    // sk_partial[tile][0 = has the tile's start, 1 = has its end][N][128], added by k_mmq_sk_fixup.
    int streamk, total_tiles;
    float *sk_partial;
};

// CTA that works on unit u when G CTAs split T units as above
__host__ __device__ inline int sk_cta_of(int64_t u, int64_t T, int G) {
    int c = (int)(u * G / T);
    while (c + 1 < G && (int64_t)(c + 1) * T / G <= u) c++;
    while (c > 0 && (int64_t)c * T / G > u) c--;
    return c;
}

constexpr int Q4K_THREADS = tc::THREADS + 32;   // the common roles plus a second MMA-issuing warp (warp 26)

// packed f32 pairs: one instruction for two columns of the epilogue
__device__ __forceinline__ uint64_t f2pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2unpack(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

template <int NPAD, int RAW_STAGES, int ACT_STAGES>
__global__ void __launch_bounds__(Q4K_THREADS, 1) k_mmq_tc_q4k(const __grid_constant__ TcMaps maps, TcParams p) {
    using namespace tc;
    constexpr int BLOB = (NPAD * 548 + 127) / 128 * 128;
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);  // f16 x f16 -> f32, K-major A and B
    // Tensor memory: the S and T accumulators of two super-blocks in [0, 4 NPAD); behind them a ring of whole
    // super-blocks of the A operand, four quarters of 32 columns (64 f16 per row) each.
    constexpr uint32_t A_COL0 = 4 * NPAD;
    constexpr int RING = (int)(TMEM_COLS - A_COL0) / 128;   // super-blocks in the ring: 3 (2 for 64 columns)
    // (d, dmin) and the mins operand are kept for eight super-blocks. Nobody waits before overwriting an entry:
    // the set that writes super-block i waited, two super-blocks earlier, for the MMAs of i - 5 to finish (its ring
    // slot), those were issued only after the epilogue of i - 7 had read its entry, and the epilogue works in order.
    constexpr int META = 8;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (tc::su32(smem_raw) & 1023u)) & 1023u);   // 1 KB of slack is allocated for this
    uint8_t *raw = smem;                                   // RAW_STAGES x RAW_BYTES
    uint8_t *actb = raw + RAW_STAGES * RAW_BYTES;          // ACT_STAGES x BLOB
    uint8_t *amin = actb + ACT_STAGES * BLOB;              // META x AMIN_BYTES
    float2 *dd = reinterpret_cast<float2 *>(amin + META * AMIN_BYTES);  // [META][ROWS] (d, dmin)
    __shared__ uint64_t bar_raw[RAW_STAGES], bar_act[ACT_STAGES], bar_afree[RING], bar_mma[2], bar_epi[4], bar_aready[RING], bar_rawfree[RAW_STAGES],
        bar_actfree[ACT_STAGES];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_fail;
    volatile int *fail = &s_fail;

    const int tid = threadIdx.x, warp = tid >> 5;
    // This CTA's units of the flattened (row tile, super-block) space: one K range of one tile (grid = tiles x
    // splits), or with stream-K an equal share of all units.
    const int split = p.streamk ? 0 : blockIdx.y;
    int64_t u0;
    int nsb;   // units of this CTA
    if (p.streamk) {
        const int64_t T = (int64_t)p.total_tiles * p.nsb;
        u0 = (int64_t)blockIdx.x * T / gridDim.x;
        nsb = (int)((int64_t)(blockIdx.x + 1) * T / gridDim.x - u0);
    } else {
        const int sb0 = split * p.sb_per_split;
        u0 = (int64_t)blockIdx.x * p.nsb + sb0;
        nsb = min(p.sb_per_split, p.nsb - sb0);            // >= 1 by construction
    }
    const int64_t u1 = u0 + nsb;
    // matrix and row tile of a global tile index (selected with constant indices: indexing kernel parameters
    // with a run-time value makes the compiler copy them to local memory, and a tensor map must stay in
    // parameter space)
    auto mat_of = [&](int gtile) { return (p.n_mats > 1 && gtile >= p.tile0[1]) + (p.n_mats > 2 && gtile >= p.tile0[2]); };
    auto tile_in_mat = [&](int gtile, int mat) { return gtile - (mat == 0 ? 0 : (mat == 1 ? p.tile0[1] : p.tile0[2])); };
    if (tid == 0) {
        for (int i = 0; i < RAW_STAGES; i++) {
            mbar_init(&bar_raw[i], 1);
            mbar_init(&bar_rawfree[i], 8);    // one arrival per warp of the set that expands this super-block
        }
        for (int i = 0; i < ACT_STAGES; i++) {
            mbar_init(&bar_act[i], 1);
            mbar_init(&bar_actfree[i], 256);
        }
        for (int i = 0; i < 2; i++) mbar_init(&bar_mma[i], 1);
        for (int i = 0; i < 4; i++) mbar_init(&bar_epi[i], 256);
        for (int i = 0; i < RING; i++) {
            mbar_init(&bar_afree[i], 1);
            mbar_init(&bar_aready[i], 8);   // the eight warps of the set that expands this super-block
        }
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&tmem_base_s, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // (tile, super-block) of the first unit; the loaders and the epilogue walk on from there without divisions
    const int tile_first = (int)(u0 / p.nsb), sb_first = (int)(u0 - (int64_t)tile_first * p.nsb);
    int lr_tile = tile_first, lr_sb = sb_first, la_sb = sb_first;   // next unit of load_raw / load_act (one thread each)
    auto load_raw = [&](int i) {   // unit i of this CTA -> raw stage i % RAW_STAGES; called for i = 0, 1, 2, ...
        const int s = i % RAW_STAGES;
        const int mat = mat_of(lr_tile);
        const CUtensorMap *wmap = mat == 0 ? &maps.m[0] : (mat == 1 ? &maps.m[1] : &maps.m[2]);
        mbar_expect_tx(&bar_raw[s], RAW_BYTES);
        tma_2d(raw + s * RAW_BYTES, wmap, lr_sb * 144, tile_in_mat(lr_tile, mat) * ROWS, &bar_raw[s]);
        if (++lr_sb == p.nsb) {
            lr_sb = 0;
            lr_tile++;
        }
    };
    auto load_act = [&](int i) {   // called for i = 0, 1, 2, ...
        const int s = i % ACT_STAGES;
        mbar_expect_tx(&bar_act[s], BLOB);
        bulk_g2s(actb + s * BLOB, p.act + (size_t)la_sb * BLOB, BLOB, &bar_act[s]);
        if (++la_sb == p.nsb) la_sb = 0;
    };
    // the weights do not depend on the kernel before this one: their first loads go out before the
    // dependency wait; activations (and everything downstream of them) come after it
    griddep_launch();
    if (tid == 0)
        for (int i = 0; i < nsb && i < RAW_STAGES; i++) load_raw(i);
    griddep_wait();
    if (tid == 0)
        for (int i = 0; i < nsb && i < ACT_STAGES; i++) load_act(i);

    // ---- warp roles: no CTA-wide barrier inside the loop, the roles meet only through mbarriers
    //   warp 0, lane 0      issues the TMA copies
    //   warps 25, 26        issue the MMAs of alternate super-blocks (one elected lane each)
    //   warps 1..8          epilogue: TMEM -> registers, f32 scaling, final store (lane quadrant = warp % 4,
    //                       two warps per quadrant split the columns)
    //   warps 9..24         expand the raw nibbles into the f16 operand (two sets of eight warps on alternate
    //                       super-blocks; see there)
    const int lane = tid & 31;
    if (warp == 0) {
        // ---- TMA producer: refills a raw stage once every expanding warp has left it, and an
        // activation stage once the epilogue of its super-block has read its scales
        if (lane == 0) {
            for (int i = 0; i < nsb; i++) {
                if (i + RAW_STAGES < nsb) {
                    mbar_wait_nap(&bar_rawfree[i % RAW_STAGES], (uint32_t)((i / RAW_STAGES) & 1), fail, 64);
                    load_raw(i + RAW_STAGES);
                }
                if (i >= 1 && i - 1 + ACT_STAGES < nsb) {
                    mbar_wait_nap(&bar_actfree[(i - 1) % ACT_STAGES], (uint32_t)(((i - 1) / ACT_STAGES) & 1), fail, 64);
                    load_act(i - 1 + ACT_STAGES);
                }
            }
        }
    } else if (warp >= MMA_WARP) {
        // ---- MMA issuers: nothing but waits on operands and tcgen05.mma / commit. Two warps take alternate
        // super-blocks: the waits of one (each costs 100 to 300 cycles even when the barrier has long completed)
        // run while the other one's instructions keep the tensor pipe busy. A whole warp runs the loop (converged,
        // so the descriptor arithmetic stays on the uniform datapath); one elected lane issues. The accumulator
        // buffer (i & 1) and the mins operand belong to one warp each, and a commit covers the MMAs of its own thread.
        const bool leader = elect_one();
        const int w = warp - MMA_WARP;
        int ring_u = w % RING;
        uint32_t ring_ph = (uint32_t)((w / RING) & 1);
        for (int i = w; i < nsb; i += 2) {
            const int as = i % ACT_STAGES, mt = i & (META - 1);
            const uint32_t d_S = tmem_base + (uint32_t)(w * 2 * NPAD), d_T = d_S + NPAD;
            const uint64_t b_desc0 = smem_desc(su32(actb + as * BLOB), 128, 4096);
            const uint64_t am_desc = smem_desc(su32(amin + mt * AMIN_BYTES), 128, 256);
            const uint64_t bm_desc = smem_desc(su32(actb + as * BLOB + NPAD * 512), 128, 256);
            const uint32_t ta0 = tmem_base + A_COL0 + (uint32_t)(ring_u * 128);   // 16 K chunks x 8 columns
            mbar_wait_nap(&bar_act[as], (uint32_t)((i / ACT_STAGES) & 1), fail, 32);
            if (i >= 2) mbar_wait_nap(&bar_epi[(i - 2) & 3], (uint32_t)(((i - 2) >> 2) & 1), fail, 32);   // TMEM buffer drained
            mbar_wait_nap(&bar_aready[ring_u], ring_ph, fail, 32);
            tc_fence_after();
            if (leader) {
                umma_f16(d_T, am_desc, bm_desc, IDESC, 0u);
#pragma unroll
                for (int kc = 0; kc < 16; kc++) umma_f16_ta(d_S, ta0 + (uint32_t)(kc * 8), b_desc0 + (uint64_t)(kc * 16), IDESC, kc ? 1u : 0u);
                umma_commit(&bar_afree[ring_u]);
                umma_commit(&bar_mma[w]);
            }
            __syncwarp();
            ring_u += 2;
            if (ring_u >= RING) {
                ring_u -= RING;
                ring_ph ^= 1u;
            }
        }
    } else if (warp < DEQ_WARP0) {
        const int q = warp & 3;                 // TMEM lane quadrant this warp may read
        const int row_in_tile = q * 32 + lane;
        constexpr int CW = NPAD / 2;            // columns of this warp
        const int col0 = ((warp - EPI_WARP0) >> 2) * CW;
        uint64_t yacc[CW / 2];                  // two columns per register pair
#pragma unroll
        for (int c = 0; c < CW / 2; c++) yacc[c] = 0ull;
        // the sums of a finished tile go out: to y, to the K-split partial sums, or (stream-K, tile cut by a CTA
        // boundary) to one of the tile's two stream-K partial results
        auto store_tile = [&](int gtile) {
            const int mat = mat_of(gtile);
            const int64_t M_mat = mat == 0 ? p.M[0] : (mat == 1 ? p.M[1] : p.M[2]);
            float *out_mat = mat == 0 ? p.out[0] : (mat == 1 ? p.out[1] : p.out[2]);
            const int64_t row = (int64_t)tile_in_mat(gtile, mat) * ROWS + row_in_tile;
            const int64_t t0 = (int64_t)gtile * p.nsb;
            float *o;
            int64_t ldo;
            if (p.streamk && (t0 < u0 || t0 + p.nsb > u1)) {
                o = p.sk_partial + ((size_t)gtile * 2 + (t0 >= u0 ? 0 : 1)) * p.N * ROWS + row_in_tile;
                ldo = ROWS;
            } else if (row < M_mat) {
                // partial sums [split][N][M] and the outputs of a group are dense; a single matrix may have its own stride
                ldo = (p.n_split > 1 || p.n_mats > 1) ? M_mat : p.ldy;
                o = out_mat + (size_t)split * p.N * ldo + row;
            } else {
                return;
            }
#pragma unroll
            for (int c = 0; c < CW / 2; c++) {
                float v0, v1;
                f2unpack(yacc[c], v0, v1);
                if (col0 + 2 * c < p.N) o[(size_t)(col0 + 2 * c) * ldo] = v0;
                if (col0 + 2 * c + 1 < p.N) o[(size_t)(col0 + 2 * c + 1) * ldo] = v1;
            }
        };
        int cur_tile = tile_first, e_sb = sb_first;
        for (int i = 0; i < nsb; i++) {
            const int b = i & 1, mt = i & (META - 1);
            if (e_sb == p.nsb) {   // stream-K only: the previous unit was the last one of its tile
                store_tile(cur_tile);
#pragma unroll
                for (int c = 0; c < CW / 2; c++) yacc[c] = 0ull;
                cur_tile++;
                e_sb = 0;
            }
            e_sb++;
            mbar_wait_nap(&bar_mma[b], (uint32_t)((i >> 1) & 1), fail, 64);
            tc_fence_after();
            const float2 sc = dd[mt * ROWS + row_in_tile];
            const float2 *yd = reinterpret_cast<const float2 *>(actb + (i % ACT_STAGES) * BLOB + NPAD * 544) + (col0 >> 1);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * 2 * NPAD + col0);
            // all loads are in flight before the one wait; the TMEM buffer is handed back as soon as
            // the values sit in registers, before the arithmetic
            float S[CW], T[CW];
            if constexpr (CW == 8) {
                tmem_ld8(lane_addr, *reinterpret_cast<float(*)[8]>(&S[0]));
                tmem_ld8(lane_addr + NPAD, *reinterpret_cast<float(*)[8]>(&T[0]));
            } else {
#pragma unroll
                for (int c = 0; c < CW; c += 16) {
                    tmem_ld16(lane_addr + c, *reinterpret_cast<float(*)[16]>(&S[c]));
                    tmem_ld16(lane_addr + NPAD + c, *reinterpret_cast<float(*)[16]>(&T[c]));
                }
            }
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&bar_epi[i & 3]);   // TMEM buffer b may be reused
            const float ds = sc.x * 16384.f;   // the weight operand carries 2^-14
            const uint64_t d2 = f2pack(ds, ds), m2 = f2pack(-sc.y, -sc.y);
#pragma unroll
            for (int c = 0; c < CW / 2; c++) {
                const float2 y2 = yd[c];
                // yd * (d * S - dmin * T), two columns per instruction
                const uint64_t t = f2fma(m2, f2pack(T[2 * c], T[2 * c + 1]), f2mul(d2, f2pack(S[2 * c], S[2 * c + 1])));
                yacc[c] = f2fma(f2pack(y2.x, y2.y), t, yacc[c]);
            }
            mbar_arrive(&bar_actfree[i % ACT_STAGES]);
        }
        store_tile(cur_tile);
    } else {
        // Two sets of eight warps take alternate super-blocks (set 0 the even ones of this CTA, set 1 the odd ones), so
        // a warp's chain of barrier waits, shared-memory loads, TMEM stores and arrivals (several hundred cycles of
        // latency that nothing in the same warp can hide) is paid once per TWO super-blocks of CTA progress, and the
        // two sets are half a period apart. Inside a set: lane quadrant = warp % 4 (a warp may only touch the 32
        // TMEM lanes of its quadrant), half = which two 32-byte qs chunks (quarters of the super-block) of its
        // row the thread expands.
        const int e = warp - DEQ_WARP0;
        const int q = warp & 3;                            // lane quadrant
        const int half = (e >> 2) & 1;                     // quarters 2 half and 2 half + 1
        const int set = e >> 3;
        const int r = q * 32 + lane;                       // row
        const uint32_t a_lane = tmem_base + A_COL0 + ((uint32_t)(q * 32) << 16);
        const __half2 k1024 = __half2(__ushort_as_half(0x6400), __ushort_as_half(0x6400));
        // The two quarters of a super-block are published (their barriers arrived on) only after the first values of
        // the set's NEXT super-block have been computed, so the latency of the TMEM stores hides behind arithmetic;
        // a set's first super-block is published at once so that the first MMA starts early, its last one after
        // the loop.
        int pend = -1;   // ring slot (super-block) with stores in flight
        auto publish = [&]() {
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_aready[pend]);
            pend = -1;
        };
        int ru = set % RING, rs = set % RAW_STAGES;        // ring slot and raw stage of super-block i, and their phases
        uint32_t ring_ph = (uint32_t)((set / RING) & 1), raw_ph = 0;
        for (int i = set; i < nsb; i += 2) {
            mbar_wait(&bar_raw[rs], raw_ph, fail);
            const uint8_t *rrow = raw + rs * RAW_BYTES + r * 144;
            const uint4 hdr = *reinterpret_cast<const uint4 *>(rrow);
            uint4 wv[4];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = *reinterpret_cast<const uint4 *>(rrow + 16 + half * 64 + j * 16);
            // 6-bit scales of the eight sub-blocks (get_scale_min_k4, ggml-quants.c:880-887): this thread's four
            // (sub-blocks 4 half ... 4 half + 3) as the bytes of one word
            const uint32_t sc4 = half == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u));
            if (half == 0) {
                // (d, dmin) for the epilogue and the mins as the f16 operand of the T product
                const int mt = i & (META - 1);
                dd[mt * ROWS + r] = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
                uint32_t mn8[2];
                mn8[0] = hdr.z & 0x3f3f3f3fu;
                mn8[1] = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
                uint8_t *am = amin + mt * AMIN_BYTES + (r >> 3) * 256 + (r & 7) * 16;
#pragma unroll
                for (int kc = 0; kc < 2; kc++) {
                    // small integer -> f16 without a conversion: bytes (m, 0x64) are the f16 1024 + m
                    uint32_t hm[4];
                    uint32_t t0 = __byte_perm(mn8[kc], 0x64646464u, 0x4140), t1 = __byte_perm(mn8[kc], 0x64646464u, 0x4342);
                    const __half2 v0 = __hsub2(*reinterpret_cast<__half2 *>(&t0), k1024), v1 = __hsub2(*reinterpret_cast<__half2 *>(&t1), k1024);
                    // a min multiplies the two 16-value bsums of its sub-block: each one fills a pair of K slots
                    const uint32_t p0 = *reinterpret_cast<const uint32_t *>(&v0), p1 = *reinterpret_cast<const uint32_t *>(&v1);
                    hm[0] = __byte_perm(p0, p0, 0x1010);
                    hm[1] = __byte_perm(p0, p0, 0x3232);
                    hm[2] = __byte_perm(p1, p1, 0x1010);
                    hm[3] = __byte_perm(p1, p1, 0x3232);
                    *reinterpret_cast<uint4 *>(am + kc * 128) = make_uint4(hm[0], hm[1], hm[2], hm[3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> async-proxy (MMA) reads
            }
#pragma unroll
            for (int qq = 0; qq < 2; qq++) {
                // quarter 2 half + qq = qs chunk of 32 bytes = sub-blocks 2 (2 half + qq) (low nibbles) and + 1 (high nibbles).
                // f16 scale pairs (sc, sc), built from the integer bytes without conversions: bytes (sc, 0x64) are the
                // f16 1024 + sc. A 4-bit code masked out of a word where it stands, (w & 0x000f) or (w & 0x00f0), is
                // the f16 SUBNORMAL q * 2^-24 or q * 2^-20; times sc * 2^10 or sc * 2^6 that is sc * q * 2^-14, a normal
                // f16 number, exactly (sc * q <= 945 has 10 bits). So a pair of weights costs one AND with an immediate
                // and one HMUL2, no constants are held in registers, and the epilogue multiplies S by 2^14.
                uint32_t tl = __byte_perm(sc4, 0x64646464u, qq ? 0x4242 : 0x4040);
                uint32_t th = __byte_perm(sc4, 0x64646464u, qq ? 0x4343 : 0x4141);
                const __half2 mlo = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&tl), k1024), __half2(__ushort_as_half(0x6400), __ushort_as_half(0x6400)));   // sc * 2^10
                const __half2 mhi = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&th), k1024), __half2(__ushort_as_half(0x5400), __ushort_as_half(0x5400)));   // sc * 2^6
                const uint32_t ws[8] = {wv[2 * qq].x, wv[2 * qq].y, wv[2 * qq].z, wv[2 * qq].w, wv[2 * qq + 1].x, wv[2 * qq + 1].y, wv[2 * qq + 1].z, wv[2 * qq + 1].w};
                const int slot = ru * 4 + 2 * half + qq;
                // 32 low-nibble values (K chunks 0 and 1 of the quarter), two per 32-bit column in the order the nibbles
                // leave a word: (0,2) (1,3) (4,6) (5,7) ...; then the 32 high-nibble values (K chunks 2 and 3)
                uint32_t v[16];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    uint32_t t0 = ws[k] & 0x000f000fu, t1 = (ws[k] >> 8) & 0x000f000fu;
                    const __half2 l0 = __hmul2(*reinterpret_cast<__half2 *>(&t0), mlo);
                    const __half2 l1 = __hmul2(*reinterpret_cast<__half2 *>(&t1), mlo);
                    v[2 * k] = *reinterpret_cast<const uint32_t *>(&l0);
                    v[2 * k + 1] = *reinterpret_cast<const uint32_t *>(&l1);
                }
                if (qq == 0) {
                    if (pend >= 0) publish();
                    if (i >= RING) {   // the MMAs that read this ring slot last time are done
                        mbar_wait(&bar_afree[ru], ring_ph ^ 1u, fail);
                        tc_fence_after();
                    }
                }
                tmem_st16(a_lane + (uint32_t)(slot * 32), v);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    uint32_t u0 = ws[k] & 0x00f000f0u, u1 = (ws[k] >> 8) & 0x00f000f0u;
                    const __half2 h0 = __hmul2(*reinterpret_cast<__half2 *>(&u0), mhi);
                    const __half2 h1 = __hmul2(*reinterpret_cast<__half2 *>(&u1), mhi);
                    v[2 * k] = *reinterpret_cast<const uint32_t *>(&h0);
                    v[2 * k + 1] = *reinterpret_cast<const uint32_t *>(&h1);
                }
                tmem_st16(a_lane + (uint32_t)(slot * 32 + 16), v);
            }
            pend = ru;
            if (i < 2) publish();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_rawfree[rs]);
            ru += 2;
            if (ru >= RING) {
                ru -= RING;
                ring_ph ^= 1u;
            }
            rs += 2;
            if (rs >= RAW_STAGES) {
                rs -= RAW_STAGES;
                raw_ph ^= 1u;
            }
        }
        if (pend >= 0) publish();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
    if (tid == 0 && s_fail) atomicExch(p.err, 2);
}

// y[n][m] = sum over the K splits, in split order. Up to three matrices per launch: element i of the
// concatenated index space belongs to the first segment whose end exceeds it; segment j has `seg_n[j]`
// elements, partial sums at part + seg_off[j] laid out [split][seg_n[j]], result y[j].
struct ReduceSegs {
    float *y[TC_MAX_MATS];
    int64_t seg_n[TC_MAX_MATS], seg_off[TC_MAX_MATS];
    int n_segs;
};
template <int NS>   // upper bound of n_split: exactly that many loads are issued before the first add
__global__ void __launch_bounds__(256) k_mmq_reduce(const float *__restrict__ part, ReduceSegs g, int64_t total, int n_split) {
    griddep_launch();
    griddep_wait();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    // segment of element i, chosen with constant indices into the parameter struct
    int64_t stride = g.seg_n[0], off = g.seg_off[0];
    float *__restrict__ y = g.y[0];
    if (g.n_segs > 1 && i >= g.seg_n[0]) {
        i -= g.seg_n[0];
        stride = g.seg_n[1]; off = g.seg_off[1]; y = g.y[1];
        if (g.n_segs > 2 && i >= g.seg_n[1]) {
            i -= g.seg_n[1];
            stride = g.seg_n[2]; off = g.seg_off[2]; y = g.y[2];
        }
    }
    const float *p = part + off + i;
    // all loads go out before the first add: a warp issues in order, and an add right behind its load
    // would make every L2 round trip wait for the one before it
    float v[NS];
#pragma unroll
    for (int k = 0; k < NS; k++) v[k] = k < n_split ? p[(size_t)k * stride] : 0.f;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NS; k++)
        if (k < n_split) s += v[k];
    y[i] = s;
}

// stream-K: a tile cut by a CTA boundary has two partial results; their sum (start part + end part) is the tile
struct SkFixup {
    const float *partial;
    float *y[TC_MAX_MATS];
    int64_t M[TC_MAX_MATS];
    int tile0[TC_MAX_MATS + 1];
    int n_mats, N, nsb, total_tiles, n_ctas;
};
__global__ void __launch_bounds__(256) k_mmq_sk_fixup(SkFixup f) {
    griddep_launch();
    griddep_wait();
    const int gtile = blockIdx.x;
    const int64_t T = (int64_t)f.total_tiles * f.nsb, t0 = (int64_t)gtile * f.nsb;
    if (sk_cta_of(t0, T, f.n_ctas) == sk_cta_of(t0 + f.nsb - 1, T, f.n_ctas)) return;   // one CTA had the whole tile
    const int mat = (f.n_mats > 1 && gtile >= f.tile0[1]) + (f.n_mats > 2 && gtile >= f.tile0[2]);
    const int64_t M_mat = mat == 0 ? f.M[0] : (mat == 1 ? f.M[1] : f.M[2]);
    float *y = mat == 0 ? f.y[0] : (mat == 1 ? f.y[1] : f.y[2]);
    const int64_t row0 = (int64_t)(gtile - (mat == 0 ? 0 : (mat == 1 ? f.tile0[1] : f.tile0[2]))) * tc::ROWS;
    const float *p0 = f.partial + (size_t)gtile * 2 * f.N * tc::ROWS, *p1 = p0 + (size_t)f.N * tc::ROWS;
    for (int i = threadIdx.x; i < f.N * tc::ROWS; i += blockDim.x) {
        const int n = i / tc::ROWS, r = i % tc::ROWS;
        if (row0 + r < M_mat) y[(size_t)n * M_mat + row0 + r] = p0[i] + p1[i];
    }
}

static cudaError_t launch_reduce_segs(const float *partial, const ReduceSegs &g, int64_t total, int n_split, cudaStream_t st) {
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    if (n_split <= 2) return launch_pdl(k_mmq_reduce<2>, grid, block, 0, st, partial, g, total, n_split);
    if (n_split <= 4) return launch_pdl(k_mmq_reduce<4>, grid, block, 0, st, partial, g, total, n_split);
    if (n_split <= 8) return launch_pdl(k_mmq_reduce<8>, grid, block, 0, st, partial, g, total, n_split);
    return launch_pdl(k_mmq_reduce<16>, grid, block, 0, st, partial, g, total, n_split);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

template <int NPAD, int RS, int AS>
static size_t tc_smem() {
    return (size_t)RS * tc::RAW_BYTES + (size_t)AS * tc_blob_bytes(NPAD) + 8 * tc::AMIN_BYTES +
           8 * tc::ROWS * sizeof(float2) + 1024;
}

void mmq_tc_configure() {
    cudaFuncSetAttribute(k_mmq_tc_q4k<16, 6, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem<16, 6, 4>());
    cudaFuncSetAttribute(k_mmq_tc_q4k<32, 6, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem<32, 6, 4>());
    cudaFuncSetAttribute(k_mmq_tc_q4k<64, 5, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem<64, 5, 2>());
}

bool mmq_tc_supported(uint32_t type, int64_t K, int64_t M, int64_t N) {
    return type == TLB_TYPE_Q4_K && K % 256 == 0 && K >= 256 && M >= 1 && N > 4 && N <= (int64_t)MM_FOLD_NPAD * 65535 && encode_tiled() != nullptr;
}

TcPlan mmq_tc_plan(int64_t K, int64_t M, int64_t N, int sm_count) {
    TcPlan t;
    t.nsb = (int)(K / 256);
    if (N > 64 && !getenv("TLB_PROMPT_EXACT")) {
        // prompt-sized batches: the folded-scale GEMM of k_mmq_tc_q8.cu (weights dequantized to f16 in the kernel, one
        // accumulator per 128 x 256 tile) instead of 64-column chunks with the reference's integer sums
        t.npad = MM_FOLD_NPAD;
        t.n_split = 1;
        t.sb_per_split = t.nsb;
        t.streamk = 0;
        t.n_col_chunks = (int)((N + t.npad - 1) / t.npad);
        t.blob_unit = mm_fold_blob_unit();
        t.blob_bytes = (uint64_t)t.n_col_chunks * t.nsb * t.blob_unit;
        t.partial_bytes = 0;
        return t;
    }
    t.npad = N <= 16 ? 16 : (N <= 32 ? 32 : 64);
    const int64_t tiles = (M + tc::ROWS - 1) / tc::ROWS;
    // K split: modelled time = waves x (CTA start-up and tail + super-blocks per CTA x time per super-block)
    // + the reduce launch when split; constants measured on B200 (3.4 us start-up and tail, 0.66 us per
    // super-block, 2 us for the reduce)
    int best = 1;
    double best_score = 1e30;
    for (int s = 1; s <= t.nsb && s <= 16; s++) {
        const int per = (t.nsb + s - 1) / s;
        if (s > 1 && per < 2) break;
        const int splits = (t.nsb + per - 1) / per;
        if (splits != s) continue;
        const int64_t units = tiles * splits;
        const int64_t waves = (units + sm_count - 1) / sm_count;
        const double score = (double)waves * (3.4 + 0.66 * per) + (splits > 1 ? 2.0 : 0.0);
        if (score < best_score) { best_score = score; best = splits; }
    }
    t.n_split = best;
    t.sb_per_split = (t.nsb + best - 1) / best;
    // stream-K when the tiles make several waves: start-up and tail + units per CTA + 2.5 us fix-up, against whole
    // waves of tiles. Measured on B200: [128256 x 4096] x 32 (6.8 waves) 144 -> 126 us; gate + up of an 8B layer
    // as one launch (1.5 waves) came out 3 us SLOWER per layer than two launches, hence the floor of 2.5 waves.
    t.streamk = 0;
    if (tiles * 2 >= (int64_t)sm_count * 5 && N <= t.npad && !getenv("TLB_NO_STREAMK")) {
        const double sk = 3.4 + (double)((tiles * t.nsb + sm_count - 1) / sm_count) * 0.66 + 2.5;
        if (sk < best_score) {
            t.streamk = sm_count;
            t.n_split = 1;
            t.sb_per_split = t.nsb;
        }
    }
    t.n_col_chunks = (int)((N + t.npad - 1) / t.npad);
    t.blob_unit = (uint64_t)tc_blob_bytes(t.npad);
    t.blob_bytes = (uint64_t)t.n_col_chunks * t.nsb * t.blob_unit;
    t.partial_bytes = t.streamk ? (uint64_t)tiles * 2 * std::min<int64_t>(N, t.npad) * tc::ROWS * 4
                                : (t.n_split > 1 ? (uint64_t)t.n_split * std::min<int64_t>(N, t.npad) * M * 4 : 0);
    return t;
}

cudaError_t launch_act_pack_tc(const ActLayout &a, const void *act, int npad, void *blobs, cudaStream_t st) {
    if (npad == MM_FOLD_NPAD) return launch_act_pack_fold(a, act, blobs, st);
    const char *ab = (const char *)act;
    k_act_pack_tc<<<dim3((unsigned)(a.K / 256), (unsigned)((a.N + npad - 1) / npad)), 256, 0, st>>>((const int8_t *)(ab + a.qs_off), (const float *)(ab + a.d_off),
                                                        (const int16_t *)(ab + a.bsum_off), a.K, (int)a.N, npad, (uint8_t *)blobs);
    return cudaGetLastError();
}

// 2-D tensor map over a row-major byte matrix (rows x row_bytes), box box_bytes x box_rows, described in
// elements of elem_bytes (1 or 2) because a box dimension may not exceed 256 elements
cudaError_t tc_encode_2d(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes, uint32_t box_rows,
                         uint32_t elem_bytes) {
    if (encode_tiled() == nullptr) return cudaErrorNotSupported;
    const cuuint64_t gdim[2] = {(cuuint64_t)(row_bytes / elem_bytes), (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {box_bytes / elem_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    if (encode_tiled()(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim,
                       gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    return cudaSuccess;
}

void launch_mmq_reduce(const float *partial, float *y, int64_t total, int n_split, cudaStream_t st) {
    ReduceSegs g{};
    g.n_segs = 1;
    g.y[0] = y;
    g.seg_n[0] = total;
    g.seg_off[0] = 0;
    launch_reduce_segs(partial, g, total, n_split, st);
}

bool tc_available() { return encode_tiled() != nullptr; }

// Test hook: every thread of one CTA waits, with the kernels' own bounded wait, on a barrier that nothing ever
// arrives on. After `limit` probes the wait gives up, the error word is set the way the mul_mat kernels set it,
// and the kernel returns; *ns receives how long thread 0 waited (globaltimer).
__global__ void k_wait_runs_out(uint32_t limit, unsigned nap_ns, int *err, unsigned long long *ns) {
    __shared__ uint64_t bar;
    __shared__ int s_fail;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    tc::mbar_wait_nap(&bar, 0u, &s_fail, nap_ns, limit);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    __syncthreads();
    if (threadIdx.x == 0) {
        *ns = t1 - t0;
        if (s_fail) atomicExch(err, 2);
    }
}
cudaError_t launch_wait_runs_out(uint32_t limit, unsigned nap_ns, int *err, unsigned long long *ns, cudaStream_t st) {
    k_wait_runs_out<<<1, 64, 0, st>>>(limit, nap_ns, err, ns);
    return cudaGetLastError();
}

// n_mats weight matrices [M[j] x K] sharing the activations; y[j] dense [N][M[j]] when n_mats > 1 or K is split
cudaError_t launch_mmq_tc_group(const TcPlan &t, int n_mats, const void *const *W, int64_t K, const int64_t *M, int64_t N, const void *blobs,
                                float *const *y, int64_t ldy, void *partial, int *err, cudaStream_t st, bool leave_partial) {
    if (t.npad == MM_FOLD_NPAD) {
        if (n_mats != 1) return cudaErrorInvalidValue;
        return launch_mm_fold_f16(true, W[0], K, M[0], N, blobs, y[0], ldy, err, st);
    }
    if (n_mats < 1 || n_mats > TC_MAX_MATS || (n_mats > 1 && t.n_col_chunks != 1)) return cudaErrorInvalidValue;
    if (t.n_split > 16) return cudaErrorInvalidValue;
    TcMaps maps;
    int tiles = 0;
    TcParams base{};
    for (int j = 0; j < n_mats; j++) {
        cudaError_t e = tc_encode_2d(&maps.m[j], W[j], (uint64_t)(K / 256 * 144), (uint64_t)M[j], 144, tc::ROWS, 1);
        if (e != cudaSuccess) return e;
        base.tile0[j] = tiles;
        base.M[j] = M[j];
        tiles += (int)((M[j] + tc::ROWS - 1) / tc::ROWS);
    }
    for (int j = n_mats; j < TC_MAX_MATS; j++) maps.m[j] = maps.m[0];
    for (int j = n_mats; j <= TC_MAX_MATS; j++) base.tile0[j] = tiles;
    base.n_mats = n_mats;
    base.npad = t.npad;
    base.nsb = t.nsb;
    base.sb_per_split = t.sb_per_split;
    base.n_split = t.n_split;
    base.err = err;
    base.ldy = ldy;
    base.total_tiles = tiles;
    base.streamk = t.streamk;
    base.sk_partial = (float *)partial;
    if (t.streamk && (t.n_split != 1 || t.n_col_chunks != 1 || (int64_t)tiles * t.nsb / t.streamk < t.nsb)) return cudaErrorInvalidValue;
    dim3 grid(t.streamk ? (unsigned)t.streamk : (unsigned)tiles, (unsigned)t.n_split);
    cudaError_t e = cudaSuccess;
    // more columns than one launch takes (prefill): one launch per chunk of npad columns
    for (int c = 0; c < t.n_col_chunks; c++) {
        const int64_t n0 = (int64_t)c * t.npad, nc = std::min<int64_t>(t.npad, N - n0);
        TcParams p = base;
        p.act = (const uint8_t *)blobs + (size_t)c * t.nsb * t.blob_unit;
        p.N = (int)nc;
        ReduceSegs segs{};
        int64_t poff = 0, total = 0;
        for (int j = 0; j < n_mats; j++) {
            float *yc = y[j] + n0 * (n_mats > 1 ? M[j] : ldy);
            if (t.n_split > 1) {
                p.out[j] = (float *)partial + poff;
                segs.y[j] = yc;
                segs.seg_n[j] = nc * M[j];
                segs.seg_off[j] = poff;
                poff += (int64_t)t.n_split * nc * M[j];
                total += nc * M[j];
            } else {
                p.out[j] = yc;
            }
        }
        switch (t.npad) {
            case 16: e = launch_pdl(k_mmq_tc_q4k<16, 6, 4>, grid, dim3(Q4K_THREADS), tc_smem<16, 6, 4>(), st, maps, p); break;
            case 32: e = launch_pdl(k_mmq_tc_q4k<32, 6, 4>, grid, dim3(Q4K_THREADS), tc_smem<32, 6, 4>(), st, maps, p); break;
            default: e = launch_pdl(k_mmq_tc_q4k<64, 5, 2>, grid, dim3(Q4K_THREADS), tc_smem<64, 5, 2>(), st, maps, p); break;
        }
        if (e != cudaSuccess) return e;
        if (t.streamk) {
            SkFixup f{};
            f.partial = (const float *)partial;
            for (int j = 0; j < n_mats; j++) {
                f.y[j] = y[j];
                f.M[j] = M[j];
            }
            for (int j = 0; j <= TC_MAX_MATS; j++) f.tile0[j] = base.tile0[j];
            f.n_mats = n_mats;
            f.N = (int)nc;
            f.nsb = t.nsb;
            f.total_tiles = tiles;
            f.n_ctas = t.streamk;
            if (n_mats == 1 && ldy != M[0]) return cudaErrorInvalidValue;   // the fix-up writes dense columns
            e = launch_pdl(k_mmq_sk_fixup, dim3((unsigned)tiles), dim3(256), 0, st, f);
            if (e != cudaSuccess) return e;
        }
        if (t.n_split > 1 && !leave_partial) {
            if (n_mats == 1 && ldy != M[0]) return cudaErrorInvalidValue;   // the reduce writes dense columns
            segs.n_segs = n_mats;
            e = launch_reduce_segs((const float *)partial, segs, total, t.n_split, st);
            if (e != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

cudaError_t launch_mmq_tc(const TcPlan &t, const void *W, int64_t K, int64_t M, int64_t N, const void *blobs, float *y,
                          int64_t ldy, void *partial, int *err, cudaStream_t st, bool leave_partial) {
    const void *Ws[1] = {W};
    float *ys[1] = {y};
    return launch_mmq_tc_group(t, 1, Ws, K, &M, N, blobs, ys, ldy, partial, err, st, leave_partial);
}

}  // namespace tlb
