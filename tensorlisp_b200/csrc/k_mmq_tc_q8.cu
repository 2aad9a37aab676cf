// Batched MUL_MAT (5 activation columns and up) with Q8_0 weights on the 5th-generation tensor cores:
// the output projection of a decode step (vocab x d_model, Q8_0) is the largest matrix of the model.
//
// Arithmetic (same integers as the reference's ggml-cpu path, vendor/ggml/src/ggml-cpu/quants.c:451-479):
// per 32-element block b, output row r and activation column c
//     D_b = sum_k q[r,k] * q8[k,c]            (int8 x int8 -> int32, exact)
//     y  += (float)D_b * (d_w[r,b] * d_a[c,b])
// tcgen05.mma kind::i8 computes D_b for 128 rows x N columns in one instruction (K = 32 = one block),
// each block into its own TMEM accumulator; the epilogue warps apply the two f32 scales.
//
// Data movement: TMA brings a 128-row x 272-byte box (8 blocks of 34 bytes per row) of raw weights and
// one packed activation blob per 256 elements of K into shared memory. The weight codes need no
// arithmetic at all: sixteen warps strip the 2-byte scales, realign the codes and store them into
// tensor memory (tcgen05.st), where the MMA reads its A operand; B (the int8 activations, K-major core
// matrices) stays in shared memory. Eight warps drain the accumulators, one warp issues the MMAs,
// one the TMA copies; they meet only through mbarriers, every wait is bounded.
#include <algorithm>
#include <cstdlib>
#include <cuda.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "tc_common.cuh"
#include "pdl.cuh"

namespace tlb {

namespace tc8 {
constexpr int ROWS = 128;
constexpr int THREADS = 832;   // TMA warp + 8 epilogue warps + 16 realigning warps + MMA warp
constexpr int EPI_WARP0 = 1, DEQ_WARP0 = 9, MMA_WARP = 25;
constexpr int STAGE_BLOCKS = 8;                       // Q8_0 blocks of a row per pipeline stage (256 elements of K)
constexpr int ROW_CHUNK = STAGE_BLOCKS * 34;          // 272 bytes: 17 x 16, so 128-bit reads at row stride are conflict-free
constexpr int RAW_BYTES = ROWS * ROW_CHUNK;
constexpr uint32_t TMEM_COLS = 512;                   // accumulators in [0, 256), the A ring in [256, 512)
constexpr uint32_t A_COL0 = 256;
constexpr int A_RING = 4;                             // stages of A (8 blocks x 8 columns of 4 int8) and of weight scales
}  // namespace tc8

// Bytes of one packed activation blob (256 elements of K, NPAD columns):
//   B    int8 [NPAD x 256]  K-major core matrices (8 columns x 16 bytes), lbo 128, sbo 2048     NPAD*256
//   d_a  f32  [8][NPAD]     activation scale per block and column                              NPAD*32
static inline __host__ __device__ int tc8_blob_bytes(int npad) { return npad * 288; }

__global__ void __launch_bounds__(256) k_act_pack_q80(const int8_t *__restrict__ qs, const float *__restrict__ ds, int64_t K, int N,
                                                       int npad, uint8_t *__restrict__ out) {
    // grid (stage, chunk of npad columns); blobs are laid out [chunk][stage]
    const int st = blockIdx.x;
    uint8_t *o = out + ((size_t)blockIdx.y * gridDim.x + st) * tc8_blob_bytes(npad);
    qs += (size_t)blockIdx.y * npad * K;
    ds += (size_t)blockIdx.y * npad * (K / 32);
    N = min(npad, N - (int)blockIdx.y * npad);
    for (int u = threadIdx.x; u < npad * 16; u += blockDim.x) {
        const int n = u / 16, kc = u % 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n < N) v = *reinterpret_cast<const uint4 *>(qs + (size_t)n * K + (size_t)st * 256 + kc * 16);
        *reinterpret_cast<uint4 *>(o + (size_t)(n / 8) * 2048 + kc * 128 + (n % 8) * 16) = v;
    }
    float *od = reinterpret_cast<float *>(o + (size_t)npad * 256);
    for (int u = threadIdx.x; u < npad * 8; u += blockDim.x) {
        const int b = u / npad, n = u % npad;
        od[u] = n < N ? ds[(size_t)n * (K / 32) + (size_t)st * 8 + b] : 0.f;
    }
}

struct Tc8Params {
    const uint8_t *act;
    float *out;
    int64_t M;
    int N, npad, nst, st_per_split, n_split;
    int64_t ldy;
    int *err;
};

namespace tc8 {
__device__ __forceinline__ void umma_i8_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16i(uint32_t taddr, int (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8i(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr));
}

// The two blocks (2G, 2G+1) of a row's 272-byte chunk are bytes [68G, 68G+68) = 17 words that start G
// words into a 16-byte unit; five aligned 128-bit reads cover them for every G. Block 2G has its scale
// in the low half of the first word and its codes 2 bytes in; block 2G+1 has its scale in the high half
// of word 8 and its codes word-aligned after it.
template <int G>
__device__ __forceinline__ void split_blocks(const uint8_t *row, uint32_t (&qa)[8], uint32_t (&qb)[8], float &da, float &db) {
    constexpr int U0 = (68 * G) / 16;      // first 16-byte unit
    constexpr int W0 = (68 * G) / 4 - 4 * U0;   // word of the chunk start inside it (= G)
    uint32_t w[20];
#pragma unroll
    for (int u = 0; u < 5; u++) {
        // for G = 3 the fifth unit is bytes 256..271: the last one of the row
        const uint4 v = *reinterpret_cast<const uint4 *>(row + (U0 + u) * 16);
        w[4 * u] = v.x; w[4 * u + 1] = v.y; w[4 * u + 2] = v.z; w[4 * u + 3] = v.w;
    }
    da = __half2float(__ushort_as_half((unsigned short)(w[W0] & 0xffffu)));
#pragma unroll
    for (int j = 0; j < 8; j++) qa[j] = __funnelshift_r(w[W0 + j], w[W0 + j + 1], 16);
    db = __half2float(__ushort_as_half((unsigned short)(w[W0 + 8] >> 16)));
#pragma unroll
    for (int j = 0; j < 8; j++) qb[j] = w[W0 + 9 + j];
}
}  // namespace tc8

template <int NPAD, int RAW_STAGES, int ACT_STAGES>
__global__ void __launch_bounds__(tc8::THREADS, 1) k_mmq_tc_q80(const __grid_constant__ CUtensorMap wmap, Tc8Params p) {
    using namespace tc;
    using namespace tc8;
    constexpr int ROWS = tc8::ROWS;
    constexpr int BLOB = NPAD * 288;
    // int8 x int8 -> int32, K-major A and B: c_format s32 (2) at bit 4, a/b format signed 8-bit (1) at bits 7 and 10
    constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
    constexpr int GCOLS = 4 * NPAD;   // accumulator columns of one group of four blocks
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (su32(smem_raw) & 1023u)) & 1023u);
    uint8_t *raw = smem;                                              // RAW_STAGES x RAW_BYTES
    uint8_t *actb = raw + RAW_STAGES * tc8::RAW_BYTES;                // ACT_STAGES x BLOB
    float *dw = reinterpret_cast<float *>(actb + ACT_STAGES * BLOB);  // [A_RING][8][ROWS] weight scales
    __shared__ uint64_t bar_raw[RAW_STAGES], bar_rawfree[RAW_STAGES], bar_act[ACT_STAGES], bar_actfree[ACT_STAGES];
    __shared__ uint64_t bar_aready[tc8::A_RING], bar_afree[tc8::A_RING], bar_dwfree[tc8::A_RING], bar_mma[2], bar_epi[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_fail;
    volatile int *fail = &s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_tile = blockIdx.x, split = blockIdx.y;
    const int st0 = split * p.st_per_split;
    const int nst = min(p.st_per_split, p.nst - st0);
    if (tid == 0) {
        for (int i = 0; i < RAW_STAGES; i++) {
            mbar_init(&bar_raw[i], 1);
            mbar_init(&bar_rawfree[i], 16);
        }
        for (int i = 0; i < ACT_STAGES; i++) {
            mbar_init(&bar_act[i], 1);
            mbar_init(&bar_actfree[i], 256);
        }
        for (int i = 0; i < tc8::A_RING; i++) {
            mbar_init(&bar_aready[i], 16);
            mbar_init(&bar_afree[i], 1);
            mbar_init(&bar_dwfree[i], 256);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&bar_mma[i], 1);
            mbar_init(&bar_epi[i], 256);
        }
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&tmem_base_s, tc8::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    auto load_raw = [&](int i) {
        const int s = i % RAW_STAGES;
        mbar_expect_tx(&bar_raw[s], tc8::RAW_BYTES);
        tma_2d(raw + s * tc8::RAW_BYTES, &wmap, (st0 + i) * (tc8::ROW_CHUNK / 2), row_tile * ROWS, &bar_raw[s]);   // x in 16-bit elements
    };
    auto load_act = [&](int i) {
        const int s = i % ACT_STAGES;
        mbar_expect_tx(&bar_act[s], BLOB);
        bulk_g2s(actb + s * BLOB, p.act + (size_t)(st0 + i) * BLOB, BLOB, &bar_act[s]);
    };
    // weights first, then the dependency wait, then activations (see k_mmq_tc.cu)
    griddep_launch();
    if (tid == 0)
        for (int i = 0; i < nst && i < RAW_STAGES; i++) load_raw(i);
    griddep_wait();
    if (tid == 0)
        for (int i = 0; i < nst && i < ACT_STAGES; i++) load_act(i);

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            for (int i = 0; i < nst; i++) {
                if (i + RAW_STAGES < nst) {
                    mbar_wait_relaxed(&bar_rawfree[i % RAW_STAGES], (uint32_t)((i / RAW_STAGES) & 1), fail);
                    load_raw(i + RAW_STAGES);
                }
                if (i >= 1 && i - 1 + ACT_STAGES < nst) {
                    mbar_wait_relaxed(&bar_actfree[(i - 1) % ACT_STAGES], (uint32_t)(((i - 1) / ACT_STAGES) & 1), fail);
                    load_act(i - 1 + ACT_STAGES);
                }
            }
        }
    } else if (warp == tc8::MMA_WARP) {
        // ---- MMA issuer: the whole warp runs the loop (converged), one elected lane issues
        const bool leader = elect_one();
        for (int i = 0; i < nst; i++) {
            const int as = i % ACT_STAGES, slot = i % tc8::A_RING;
            const uint64_t b_desc0 = smem_desc(su32(actb + as * BLOB), 128, 2048);
            mbar_wait(&bar_act[as], (uint32_t)((i / ACT_STAGES) & 1), fail);
            mbar_wait(&bar_aready[slot], (uint32_t)((i / tc8::A_RING) & 1), fail);
            tc_fence_after();
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int G = 2 * i + hh, gb = G & 1;
                if (G >= 2) {
                    mbar_wait(&bar_epi[gb], (uint32_t)(((G - 2) >> 1) & 1), fail);   // accumulator group gb drained
                    tc_fence_after();
                }
                if (leader) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int blk = 4 * hh + j;
                        umma_i8_ta(tmem_base + (uint32_t)(gb * GCOLS + j * NPAD), tmem_base + tc8::A_COL0 + (uint32_t)(slot * 64 + blk * 8),
                                   b_desc0 + (uint64_t)(blk * (256 >> 4)), IDESC);
                    }
                    umma_commit(&bar_mma[gb]);
                    if (hh == 1) umma_commit(&bar_afree[slot]);
                }
                __syncwarp();
            }
        }
    } else if (warp < tc8::DEQ_WARP0) {
        // ---- epilogue: two warps per TMEM lane quadrant split the columns
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        constexpr int CW = NPAD / 2;
        const int col0 = ((warp - tc8::EPI_WARP0) >> 2) * CW;
        float yacc[CW];
#pragma unroll
        for (int c = 0; c < CW; c++) yacc[c] = 0.f;
        for (int i = 0; i < nst; i++) {
            const int as = i % ACT_STAGES, slot = i % tc8::A_RING;
            const float *da = reinterpret_cast<const float *>(actb + as * BLOB + NPAD * 256) + col0;   // [8][NPAD]
            const float *dwr = dw + (size_t)slot * 8 * ROWS + row_in_tile;
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int G = 2 * i + hh, gb = G & 1;
                mbar_wait_relaxed(&bar_mma[gb], (uint32_t)((G >> 1) & 1), fail);
                tc_fence_after();
                const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(gb * GCOLS + col0);
#pragma unroll
                for (int jp = 0; jp < 4; jp += 2) {
                    int D0[CW], D1[CW];
                    if constexpr (CW == 8) {
                        tmem_ld8i(lane_addr + jp * NPAD, *reinterpret_cast<int(*)[8]>(&D0[0]));
                        tmem_ld8i(lane_addr + (jp + 1) * NPAD, *reinterpret_cast<int(*)[8]>(&D1[0]));
                    } else {
                        tmem_ld16i(lane_addr + jp * NPAD, *reinterpret_cast<int(*)[16]>(&D0[0]));
                        tmem_ld16i(lane_addr + (jp + 1) * NPAD, *reinterpret_cast<int(*)[16]>(&D1[0]));
                    }
                    tmem_ld_wait();
                    if (jp == 2) {
                        tc_fence_before();
                        mbar_arrive(&bar_epi[gb]);   // accumulator group gb may be overwritten
                    }
                    const int b0 = 4 * hh + jp;
                    const float w0 = dwr[b0 * ROWS], w1 = dwr[(b0 + 1) * ROWS];
#pragma unroll
                    for (int c = 0; c < CW; c++) {
                        yacc[c] += (float)D0[c] * (w0 * da[b0 * NPAD + c]);
                        yacc[c] += (float)D1[c] * (w1 * da[(b0 + 1) * NPAD + c]);
                    }
                }
            }
            mbar_arrive(&bar_dwfree[slot]);
            mbar_arrive(&bar_actfree[as]);
        }
        const int64_t row = (int64_t)row_tile * ROWS + row_in_tile;
        if (row < p.M) {
            float *o = p.out + (size_t)split * p.N * p.ldy + row;
#pragma unroll
            for (int c = 0; c < CW; c++)
                if (col0 + c < p.N) o[(size_t)(col0 + c) * p.ldy] = yacc[c];
        }
    } else {
        // ---- realigning warps: lane quadrant = warp % 4 fixes the rows; per quadrant four warps take two blocks each
        const int g = (warp - tc8::DEQ_WARP0) >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t a_lane = tmem_base + tc8::A_COL0 + ((uint32_t)((warp & 3) * 32) << 16);
        for (int i = 0; i < nst; i++) {
            const int rs = i % RAW_STAGES, slot = i % tc8::A_RING;
            mbar_wait(&bar_raw[rs], (uint32_t)((i / RAW_STAGES) & 1), fail);
            const uint8_t *rrow = raw + rs * tc8::RAW_BYTES + r * tc8::ROW_CHUNK;
            uint32_t qa[8], qb[8];
            float da, db;
            switch (g) {   // warp-uniform
                case 0: split_blocks<0>(rrow, qa, qb, da, db); break;
                case 1: split_blocks<1>(rrow, qa, qb, da, db); break;
                case 2: split_blocks<2>(rrow, qa, qb, da, db); break;
                default: split_blocks<3>(rrow, qa, qb, da, db); break;
            }
            if (i >= tc8::A_RING) {
                // the MMAs that read this ring slot are done, and the epilogue has read its scales
                mbar_wait(&bar_afree[slot], (uint32_t)(((i / tc8::A_RING) - 1) & 1), fail);
                mbar_wait(&bar_dwfree[slot], (uint32_t)(((i / tc8::A_RING) - 1) & 1), fail);
                tc_fence_after();
            }
            tmem_st8(a_lane + (uint32_t)(slot * 64 + (2 * g) * 8), qa);
            tmem_st8(a_lane + (uint32_t)(slot * 64 + (2 * g + 1) * 8), qb);
            float *dws = dw + (size_t)slot * 8 * ROWS + r;
            dws[(2 * g) * ROWS] = da;
            dws[(2 * g + 1) * ROWS] = db;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_aready[slot]);
                mbar_arrive(&bar_rawfree[rs]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tc8::TMEM_COLS);
    if (tid == 0 && s_fail) atomicExch(p.err, 2);
}

// ---------------------------------------------------------------- many activation columns (prompt pass)
// Same arithmetic, a 128-row x 128-column output tile per CTA (grid: row tiles x column tiles, row tiles
// fastest so that the CTAs in flight share a few activation blobs and sweep the weights through L2).
// One MMA (128 x 128 x 32) per block into one of two accumulators; every block's accumulator has to come back
// out of tensor memory (64 KB per block and tile) and costs an int->float conversion, a scale product and an
// FMA per element. That drain bounds this kernel, not the MMA (measured: 490 us of 790 with the arithmetic
// left out, tensor pipe 7% busy), so sixteen warps drain (lane quadrant x 32-column slice, sums in registers,
// two f32 lanes per instruction), four realign the weight codes, one issues MMAs, one TMA copies; the warps
// that mostly wait nap between probes.
namespace tc8w {
constexpr int NW = 128;                                  // activation columns per tile
constexpr int EPI_WARPS = 16, DEQ_WARPS = 4;
constexpr int EPI_WARP0 = 1, DEQ_WARP0 = EPI_WARP0 + EPI_WARPS, MMA_WARP = DEQ_WARP0 + DEQ_WARPS;
constexpr int THREADS = (MMA_WARP + 1) * 32;             // 704
constexpr int RAW_STAGES = 2, ACT_STAGES = 3;
constexpr int N_ACC = 3;                                 // accumulators of NW columns in tensor memory columns [0, 384)
constexpr uint32_t A_COL0 = N_ACC * NW;                  // the A ring behind them: 2 stages x 64 columns
constexpr int A_RING = 2;
constexpr int BLOB = NW * 288;
constexpr int CW = NW / (EPI_WARPS / 4);                 // 32 columns per draining warp
// two f32 lanes per instruction (each lane rounds as the scalar instruction does)
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// y += float(D) * (w * s) for 16 columns
__device__ __forceinline__ void drain16(uint64_t *y, const int (&D)[16], uint64_t ww, const ulonglong2 *s) {
#pragma unroll
    for (int c4 = 0; c4 < 4; c4++) {
        const ulonglong2 sv = s[c4];
        y[2 * c4] = fma2(pack2((float)D[4 * c4], (float)D[4 * c4 + 1]), mul2(ww, sv.x), y[2 * c4]);
        y[2 * c4 + 1] = fma2(pack2((float)D[4 * c4 + 2], (float)D[4 * c4 + 3]), mul2(ww, sv.y), y[2 * c4 + 1]);
    }
}
}  // namespace tc8w

__global__ void __launch_bounds__(tc8w::THREADS, 1) k_mmq_tc_q80_wide(const __grid_constant__ CUtensorMap wmap, Tc8Params p) {
    using namespace tc;
    using namespace tc8w;
    constexpr int ROWS = tc8::ROWS;
    constexpr int A_RING = tc8w::A_RING;
    constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NW >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (su32(smem_raw) & 1023u)) & 1023u);
    uint8_t *raw = smem;                                              // RAW_STAGES x RAW_BYTES
    uint8_t *actb = raw + RAW_STAGES * tc8::RAW_BYTES;                // ACT_STAGES x BLOB
    float *dw = reinterpret_cast<float *>(actb + ACT_STAGES * BLOB);  // [A_RING][8][ROWS] weight scales
    __shared__ uint64_t bar_raw[RAW_STAGES], bar_rawfree[RAW_STAGES], bar_act[ACT_STAGES], bar_actfree[ACT_STAGES];
    __shared__ uint64_t bar_aready[A_RING], bar_afree[A_RING], bar_dwfree[A_RING], bar_mma[N_ACC], bar_epi[N_ACC];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_fail;
    volatile int *fail = &s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_tile = blockIdx.x, col_tile = blockIdx.y;
    const int nst = p.nst;
    const uint8_t *act = p.act + (size_t)col_tile * nst * BLOB;
    if (tid == 0) {
        for (int i = 0; i < RAW_STAGES; i++) {
            mbar_init(&bar_raw[i], 1);
            mbar_init(&bar_rawfree[i], DEQ_WARPS);
        }
        for (int i = 0; i < ACT_STAGES; i++) {
            mbar_init(&bar_act[i], 1);
            mbar_init(&bar_actfree[i], EPI_WARPS);
        }
        for (int i = 0; i < A_RING; i++) {
            mbar_init(&bar_aready[i], DEQ_WARPS);
            mbar_init(&bar_afree[i], 1);
            mbar_init(&bar_dwfree[i], EPI_WARPS);
        }
        for (int i = 0; i < N_ACC; i++) {
            mbar_init(&bar_mma[i], 1);
            mbar_init(&bar_epi[i], EPI_WARPS);   // one arrival per draining warp
        }
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&tmem_base_s, tc8::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    auto load_raw = [&](int i) {
        const int s = i % RAW_STAGES;
        mbar_expect_tx(&bar_raw[s], tc8::RAW_BYTES);
        tma_2d(raw + s * tc8::RAW_BYTES, &wmap, i * (tc8::ROW_CHUNK / 2), row_tile * ROWS, &bar_raw[s]);   // x in 16-bit elements
    };
    auto load_act = [&](int i) {
        const int s = i % ACT_STAGES;
        mbar_expect_tx(&bar_act[s], BLOB);
        bulk_g2s(actb + s * BLOB, act + (size_t)i * BLOB, BLOB, &bar_act[s]);
    };
    griddep_launch();
    if (tid == 0)
        for (int i = 0; i < nst && i < RAW_STAGES; i++) load_raw(i);
    griddep_wait();
    if (tid == 0)
        for (int i = 0; i < nst && i < ACT_STAGES; i++) load_act(i);

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            for (int i = 0; i < nst; i++) {
                if (i + RAW_STAGES < nst) {
                    mbar_wait_relaxed(&bar_rawfree[i % RAW_STAGES], (uint32_t)((i / RAW_STAGES) & 1), fail);
                    load_raw(i + RAW_STAGES);
                }
                if (i + ACT_STAGES < nst) {
                    mbar_wait_relaxed(&bar_actfree[i % ACT_STAGES], (uint32_t)((i / ACT_STAGES) & 1), fail);
                    load_act(i + ACT_STAGES);
                }
            }
        }
    } else if (warp == tc8w::MMA_WARP) {
        // ---- MMA issuer: the whole warp runs the loop (converged), one elected lane issues
        const bool leader = elect_one();
        int gb = 0;            // accumulator of block G = 8 * i + blk: G % N_ACC, in its (G / N_ACC)-th use
        uint32_t use = 0;
        for (int i = 0; i < nst; i++) {
            const int as = i % ACT_STAGES, slot = i % A_RING;
            const uint64_t b_desc0 = smem_desc(su32(actb + as * BLOB), 128, 2048);
            mbar_wait_nap(&bar_act[as], (uint32_t)((i / ACT_STAGES) & 1), fail, 32);
            mbar_wait_nap(&bar_aready[slot], (uint32_t)((i / A_RING) & 1), fail, 32);
            tc_fence_after();
#pragma unroll 1
            for (int blk = 0; blk < 8; blk++) {
                if (use > 0) {
                    mbar_wait_nap(&bar_epi[gb], (use - 1) & 1, fail, 32);   // accumulator gb drained
                    tc_fence_after();
                }
                if (leader) {
                    tc8::umma_i8_ta(tmem_base + (uint32_t)(gb * NW), tmem_base + tc8w::A_COL0 + (uint32_t)(slot * 64 + blk * 8),
                                    b_desc0 + (uint64_t)(blk * (256 >> 4)), IDESC);
                    umma_commit(&bar_mma[gb]);
                    if (blk == 7) umma_commit(&bar_afree[slot]);
                }
                __syncwarp();
                if (++gb == N_ACC) {
                    gb = 0;
                    use++;
                }
            }
        }
    } else if (warp < tc8w::DEQ_WARP0) {
        // ---- draining warps: TMEM lane quadrant warp % 4, column slice (warp - 1) / 4
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const int col0 = ((warp - tc8w::EPI_WARP0) >> 2) * CW;
        static_assert(CW == 32, "the draining loop below takes two 16-column loads per block");
        uint64_t yacc[CW / 2];
#pragma unroll
        for (int c = 0; c < CW / 2; c++) yacc[c] = 0ull;   // two +0.0f
        const uint32_t lane_addr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col0;
        int gb = 0;
        uint32_t use = 0;
        for (int i = 0; i < nst; i++) {
            const int as = i % ACT_STAGES, slot = i % A_RING;
            const float *da = reinterpret_cast<const float *>(actb + as * BLOB + NW * 256) + col0;   // [8][NW]
            const float *dwr = dw + (size_t)slot * 8 * ROWS + row_in_tile;
#pragma unroll 1
            for (int blk = 0; blk < 8; blk++) {
                mbar_wait_relaxed(&bar_mma[gb], use & 1, fail);
                tc_fence_after();
                const float w = dwr[blk * ROWS];
                const uint64_t ww = pack2(w, w);
                const ulonglong2 *dab = reinterpret_cast<const ulonglong2 *>(da + blk * NW);
                // the second load is in flight while the first half is added up
                int D0[16], D1[16];
                tc8::tmem_ld16i(lane_addr0 + (uint32_t)(gb * NW), D0);
                tmem_ld_wait();
                tc8::tmem_ld16i(lane_addr0 + (uint32_t)(gb * NW + 16), D1);
                drain16(yacc, D0, ww, dab);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_epi[gb]);   // accumulator gb may be overwritten
                drain16(yacc + 8, D1, ww, dab + 4);
                if (++gb == N_ACC) {
                    gb = 0;
                    use++;
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_dwfree[slot]);
                mbar_arrive(&bar_actfree[as]);
            }
        }
        const int64_t row = (int64_t)row_tile * ROWS + row_in_tile;
        const int ncol = min(NW, p.N - col_tile * NW);
        if (row < p.M) {
            float *o = p.out + (size_t)col_tile * NW * p.ldy + row;
#pragma unroll
            for (int c = 0; c < CW / 2; c++) {
                float lo, hi;
                asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(yacc[c]));
                if (col0 + 2 * c < ncol) o[(size_t)(col0 + 2 * c) * p.ldy] = lo;
                if (col0 + 2 * c + 1 < ncol) o[(size_t)(col0 + 2 * c + 1) * p.ldy] = hi;
            }
        }
    } else {
        // ---- realigning warps: lane quadrant = warp % 4 fixes the rows, every warp takes all eight blocks of its rows
        const int r = (warp & 3) * 32 + lane;
        const uint32_t a_lane = tmem_base + tc8w::A_COL0 + ((uint32_t)((warp & 3) * 32) << 16);
        for (int i = 0; i < nst; i++) {
            const int rs = i % RAW_STAGES, slot = i % A_RING;
            mbar_wait_nap(&bar_raw[rs], (uint32_t)((i / RAW_STAGES) & 1), fail, 128);
            if (i >= A_RING) {
                // the MMAs that read this ring slot are done, and the draining warps have read its scales
                mbar_wait_nap(&bar_afree[slot], (uint32_t)(((i / A_RING) - 1) & 1), fail, 128);
                mbar_wait_nap(&bar_dwfree[slot], (uint32_t)(((i / A_RING) - 1) & 1), fail, 128);
                tc_fence_after();
            }
            const uint8_t *rrow = raw + rs * tc8::RAW_BYTES + r * tc8::ROW_CHUNK;
            float *dws = dw + (size_t)slot * 8 * ROWS + r;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                uint32_t qa[8], qb[8];
                float da, db;
                if (g == 0) tc8::split_blocks<0>(rrow, qa, qb, da, db);
                else if (g == 1) tc8::split_blocks<1>(rrow, qa, qb, da, db);
                else if (g == 2) tc8::split_blocks<2>(rrow, qa, qb, da, db);
                else tc8::split_blocks<3>(rrow, qa, qb, da, db);
                tmem_st8(a_lane + (uint32_t)(slot * 64 + (2 * g) * 8), qa);
                tmem_st8(a_lane + (uint32_t)(slot * 64 + (2 * g + 1) * 8), qb);
                dws[(2 * g) * ROWS] = da;
                dws[(2 * g + 1) * ROWS] = db;
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bar_aready[slot]);
                mbar_arrive(&bar_rawfree[rs]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tc8::TMEM_COLS);
    if (tid == 0 && s_fail) atomicExch(p.err, 2);
}

// ---------------------------------------------------------------- many activation columns, one accumulator (prompt pass)
// The kernel above pays for the reference's arithmetic with one accumulator round trip per 32-element block. This one
// folds both scales into the operands instead and lets the tensor core add up the whole of K:
//     A[r,k] = f16(d_w[r,b] * q[r,k])        (HMUL2 of the exact code by the block's f16 scale: one rounding)
//     B[k,c] = f16(d_a[c,b] * q8[k,c])       (by the activation packer, from the same Q8_0 quantization of the activations
//                                             that the reference makes: one rounding)
//     y[r,c] = sum_k A[r,k] * B[k,c]         (tcgen05.mma kind::f16, f32 accumulator in tensor memory)
// Each product carries two f16 roundings (2^-12 relative each, independent across k), so y differs from the reference's
// integer arithmetic by about 1e-4 of max|y| at K = 4096: inside the 1e-3 bar of mul_mat, not bit-comparable. The exact
// kernel above stays reachable (TLB_PROMPT_EXACT=1).
// A persistent CTA walks (row tile, column tile) pairs, 128 weight rows x 256 activation columns each. Per 256 elements
// of K: TMA brings 128 x 272 raw bytes; eight warps strip the scales, turn the codes into scaled f16 and store them into
// tensor memory (A operand, 128 columns); the packed B arrives as four 32 KB bulk copies (64 elements of K each, core
// matrix layout); one warp issues 16 MMAs of 128 x 256 x 16. Eight warps drain the 128 x 256 accumulator once per tile.
namespace tc8f {
constexpr int NW = 256;                                  // activation columns per tile
constexpr int KS = 64;                                   // elements of K per B stage
constexpr int B_STAGE = NW * KS * 2;                     // 32 KB
constexpr int B_STAGES = 4, RAW_STAGES = 2, A_RING = 2;
constexpr int TMA_RAW_WARP = 0, TMA_B_WARP = 1, MMA_WARP = 2;   // warp 3 idles (keeps the quadrant numbering of the rest aligned)
constexpr int DEQ_WARP0 = 4, DEQ_WARPS = 8, EPI_WARP0 = 12, EPI_WARPS = 8;
constexpr int THREADS = (EPI_WARP0 + EPI_WARPS) * 32;    // 640
constexpr uint32_t ACC_COL0 = 0, A_COL0 = 256;           // accumulator [0, 256), A ring 2 x 128 columns behind it
// 4 int8 codes of a word -> two f16x2 of code * scale (exact integer first: (1024 + u) - 1152 with u = code + 128)
__device__ __forceinline__ void codes_to_f16(uint32_t w, uint32_t dd, uint32_t &lo, uint32_t &hi) {
    const uint32_t x = w ^ 0x80808080u;
    uint32_t a = __byte_perm(x, 0x64646464u, 0x4140), b = __byte_perm(x, 0x64646464u, 0x4342);
    const uint32_t k1152 = 0x64806480u;   // f16x2 (1152, 1152)
    asm("sub.f16x2 %0, %0, %1;" : "+r"(a) : "r"(k1152));
    asm("sub.f16x2 %0, %0, %1;" : "+r"(b) : "r"(k1152));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(a), "r"(dd));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(b), "r"(dd));
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
}  // namespace tc8f

// B operand of the kernel below: blobs [chunk of 256 columns][stage of 64 elements of K] x 32 KB, each
// [column / 8][8 chunks of 8 elements][column % 8][16 bytes] (K-major core matrices: lbo 128, sbo 1024), values
// f16(d_a * q8) in the order of K.
// `blk`: elements per activation scale (32 for Q8_0 activations, 256 for the Q8_K activations of Q4_K weights).
__global__ void __launch_bounds__(256) k_act_pack_q80_f16(const int8_t *__restrict__ qs, const float *__restrict__ ds, int64_t K, int N, int blk,
                                                           uint8_t *__restrict__ out) {
    const int st = blockIdx.x;   // stage of 64 elements
    uint8_t *o = out + ((size_t)blockIdx.y * gridDim.x + st) * tc8f::B_STAGE;
    const int n0 = (int)blockIdx.y * tc8f::NW;
    for (int u = threadIdx.x; u < tc8f::NW * 8; u += blockDim.x) {
        const int nl = u / 8, kc = u % 8, n = n0 + nl;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n < N) {
            const int64_t k0 = (int64_t)st * tc8f::KS + kc * 8;
            const uint2 q = *reinterpret_cast<const uint2 *>(qs + (size_t)n * K + k0);
            const float d = ds[(size_t)n * (K / blk) + k0 / blk];
            const uint32_t w[2] = {q.x, q.y};
            uint32_t h[4];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const float f0 = (float)(int8_t)(w[i] & 0xff), f1 = (float)(int8_t)((w[i] >> 8) & 0xff), f2 = (float)(int8_t)((w[i] >> 16) & 0xff),
                            f3 = (float)(int8_t)(w[i] >> 24);
                const __half2 a = __floats2half2_rn(f0 * d, f1 * d), b = __floats2half2_rn(f2 * d, f3 * d);
                h[2 * i] = *reinterpret_cast<const uint32_t *>(&a);
                h[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&b);
            }
            v = make_uint4(h[0], h[1], h[2], h[3]);
        }
        *reinterpret_cast<uint4 *>(o + (size_t)(nl / 8) * 1024 + kc * 128 + (nl % 8) * 16) = v;
    }
}

struct Tc8fParams {
    const uint8_t *act;   // packed B blobs
    float *out;
    int64_t M, ldy;
    int N, nst, row_tiles, col_tiles;
    int *err;
};

// WQ4K = false: Q8_0 weights (raw rows of 8 x 34 bytes per unit); true: Q4_K weights (one 144-byte super-block per unit:
// f16 d, dmin, twelve bytes of 6-bit scales and mins, 128 bytes of nibbles), expanded to f16(d * sc * q - dmin * m), the f32
// value that ggml's dequantizer produces (dequantize_row_q4_K, ggml-quants.c) rounded once.
template <bool WQ4K>
__global__ void __launch_bounds__(tc8f::THREADS, 1) k_mm_q80_f16(const __grid_constant__ CUtensorMap wmap, Tc8fParams p) {
    using namespace tc;
    using namespace tc8f;
    constexpr int ROWS = tc8::ROWS;
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(tc8f::NW >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);   // f16 x f16 -> f32, K-major A and B
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (su32(smem_raw) & 1023u)) & 1023u);
    constexpr int ROW_CHUNK = WQ4K ? 144 : tc8::ROW_CHUNK;   // raw bytes of a row per unit of 256 elements
    constexpr int RAW_BYTES = ROWS * ROW_CHUNK;
    uint8_t *bst = smem;                                   // tc8f::B_STAGES x tc8f::B_STAGE
    uint8_t *raw = bst + tc8f::B_STAGES * tc8f::B_STAGE;               // tc8f::RAW_STAGES x RAW_BYTES
    __shared__ uint64_t bar_raw[tc8f::RAW_STAGES], bar_rawfree[tc8f::RAW_STAGES], bar_b[tc8f::B_STAGES], bar_bfree[tc8f::B_STAGES];
    __shared__ uint64_t bar_aready[tc8f::A_RING], bar_afree[tc8f::A_RING], bar_accfull, bar_accfree;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_fail;
    volatile int *fail = &s_fail;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nst = p.nst;   // units of 256 elements of K
    const int n_tiles = p.row_tiles * p.col_tiles;
    if (tid == 0) {
        for (int i = 0; i < tc8f::RAW_STAGES; i++) {
            mbar_init(&bar_raw[i], 1);
            mbar_init(&bar_rawfree[i], tc8f::DEQ_WARPS);
        }
        for (int i = 0; i < tc8f::B_STAGES; i++) {
            mbar_init(&bar_b[i], 1);
            mbar_init(&bar_bfree[i], 1);
        }
        for (int i = 0; i < tc8f::A_RING; i++) {
            mbar_init(&bar_aready[i], tc8f::DEQ_WARPS);
            mbar_init(&bar_afree[i], 1);
        }
        mbar_init(&bar_accfull, 1);
        mbar_init(&bar_accfree, tc8f::EPI_WARPS);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&tmem_base_s, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    griddep_launch();

    if (warp == tc8f::TMA_RAW_WARP) {
        // ---- raw weights: one 128-row x 272-byte box per unit (they do not depend on the kernel in front)
        if (lane == 0) {
            uint32_t g = 0;
            for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                const int row_tile = t % p.row_tiles;
                for (int i = 0; i < nst; i++, g++) {
                    const int s = g % tc8f::RAW_STAGES;
                    if (g >= tc8f::RAW_STAGES) mbar_wait_nap(&bar_rawfree[s], ((g / tc8f::RAW_STAGES) - 1) & 1, fail, 64);
                    mbar_expect_tx(&bar_raw[s], RAW_BYTES);
                    tma_2d(raw + s * RAW_BYTES, &wmap, i * (ROW_CHUNK / 2), row_tile * ROWS, &bar_raw[s]);   // x in 16-bit elements
                }
            }
        }
    } else if (warp == tc8f::TMA_B_WARP) {
        // ---- packed activations: four 32 KB stages per unit
        if (lane == 0) {
            griddep_wait();
            uint32_t g = 0;
            for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                const int col_tile = t / p.row_tiles;
                const uint8_t *src = p.act + (size_t)col_tile * nst * 4 * tc8f::B_STAGE;
                for (int i = 0; i < nst * 4; i++, g++) {
                    const int s = g % tc8f::B_STAGES;
                    if (g >= tc8f::B_STAGES) mbar_wait_nap(&bar_bfree[s], ((g / tc8f::B_STAGES) - 1) & 1, fail, 32);
                    mbar_expect_tx(&bar_b[s], tc8f::B_STAGE);
                    bulk_g2s(bst + s * tc8f::B_STAGE, src + (size_t)i * tc8f::B_STAGE, tc8f::B_STAGE, &bar_b[s]);
                }
            }
        }
    } else if (warp == tc8f::MMA_WARP) {
        // ---- MMA issuer: the whole warp runs the loop (converged), one elected lane issues
        const bool leader = elect_one();
        uint32_t g = 0, gb = 0, it = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, it++) {
            if (it > 0) {
                mbar_wait_nap(&bar_accfree, (it - 1) & 1, fail, 32);   // the accumulator of the tile before has been drained
                tc_fence_after();
            }
            for (int i = 0; i < nst; i++, g++) {
                const int slot = g % tc8f::A_RING;
                mbar_wait_nap(&bar_aready[slot], (g / tc8f::A_RING) & 1, fail, 32);
                tc_fence_after();
                const uint32_t a0 = tmem_base + tc8f::A_COL0 + (uint32_t)(slot * 128);
#pragma unroll 1
                for (int s4 = 0; s4 < 4; s4++, gb++) {
                    const int bs = gb % tc8f::B_STAGES;
                    mbar_wait_nap(&bar_b[bs], (gb / tc8f::B_STAGES) & 1, fail, 32);
                    tc_fence_after();
                    if (leader) {
                        const uint64_t b_desc0 = smem_desc(su32(bst + bs * tc8f::B_STAGE), 128, 1024);
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            umma_f16_ta(tmem_base + tc8f::ACC_COL0, a0 + (uint32_t)((s4 * 4 + k) * 8), b_desc0 + (uint64_t)(k * 16), IDESC,
                                        (i | s4 | k) ? 1u : 0u);
                        umma_commit(&bar_bfree[bs]);
                        if (s4 == 3) {
                            umma_commit(&bar_afree[slot]);
                            if (i == nst - 1) umma_commit(&bar_accfull);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp >= tc8f::DEQ_WARP0 && warp < tc8f::EPI_WARP0) {
        // ---- expanders: lane quadrant warp % 4 fixes the rows; the two warps of a quadrant take four blocks each
        const int q = warp & 3, half = (warp - tc8f::DEQ_WARP0) >> 2;
        const int r = q * 32 + lane;
        const uint32_t a_lane = tmem_base + tc8f::A_COL0 + ((uint32_t)(q * 32) << 16);
        uint32_t g = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
            for (int i = 0; i < nst; i++, g++) {
                const int rs = g % tc8f::RAW_STAGES, slot = g % tc8f::A_RING;
                mbar_wait_nap(&bar_raw[rs], (g / tc8f::RAW_STAGES) & 1, fail, 64);
                if (g >= tc8f::A_RING) {
                    mbar_wait_nap(&bar_afree[slot], ((g / tc8f::A_RING) - 1) & 1, fail, 64);   // the MMAs that read this slot are done
                    tc_fence_after();
                }
                const uint8_t *rrow = raw + rs * RAW_BYTES + r * ROW_CHUNK;
                if constexpr (WQ4K) {
                    // this warp's half of the super-block: the 64-value groups 2 * half and 2 * half + 1 (the low nibbles of
                    // a group's 32 bytes are one sub-block, the high nibbles the next)
                    const uint4 hdr = *reinterpret_cast<const uint4 *>(rrow);   // d, dmin, scales[12]
                    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
                    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                    // byte i of scales[12], taken out of the three words with shifts (no byte array in local memory)
                    auto sb = [&](int i) -> int { return (int)(((i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w)) >> ((i & 3) * 8)) & 0xffu); };
                    auto scale_min = [&](int jj, int &sc, int &mn) {   // get_scale_min_k4 (ggml-quants.c:880-887)
                        if (jj < 4) {
                            sc = sb(jj) & 63;
                            mn = sb(jj + 4) & 63;
                        } else {
                            sc = (sb(jj + 4) & 0xF) | ((sb(jj - 4) >> 6) << 4);
                            mn = (sb(jj + 4) >> 4) | ((sb(jj) >> 6) << 4);
                        }
                    };
#pragma unroll
                    for (int gg = 0; gg < 2; gg++) {
                        const int j = half * 2 + gg;
                        int sc0, mn0, sc1, mn1;
                        scale_min(2 * j, sc0, mn0);
                        scale_min(2 * j + 1, sc1, mn1);
                        const float a0 = __fmul_rn(d, (float)sc0), b0 = __fmul_rn(dmin, (float)mn0);
                        const float a1 = __fmul_rn(d, (float)sc1), b1 = __fmul_rn(dmin, (float)mn1);
                        uint32_t lo[16], hi[16];
#pragma unroll
                        for (int u = 0; u < 2; u++) {
                            const uint4 qv = *reinterpret_cast<const uint4 *>(rrow + 16 + j * 32 + u * 16);
                            const uint32_t w4[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                            for (int wi = 0; wi < 4; wi++) {
                                const uint32_t w = w4[wi];
                                float fl[4], fh[4];
#pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    fl[e] = __fsub_rn(__fmul_rn(a0, (float)((w >> (8 * e)) & 0xF)), b0);
                                    fh[e] = __fsub_rn(__fmul_rn(a1, (float)((w >> (8 * e + 4)) & 0xF)), b1);
                                }
                                const __half2 l0 = __floats2half2_rn(fl[0], fl[1]), l1 = __floats2half2_rn(fl[2], fl[3]);
                                const __half2 h0 = __floats2half2_rn(fh[0], fh[1]), h1 = __floats2half2_rn(fh[2], fh[3]);
                                lo[(u * 4 + wi) * 2] = *reinterpret_cast<const uint32_t *>(&l0);
                                lo[(u * 4 + wi) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&l1);
                                hi[(u * 4 + wi) * 2] = *reinterpret_cast<const uint32_t *>(&h0);
                                hi[(u * 4 + wi) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&h1);
                            }
                        }
                        tmem_st16(a_lane + (uint32_t)(slot * 128 + j * 32), lo);
                        tmem_st16(a_lane + (uint32_t)(slot * 128 + j * 32 + 16), hi);
                    }
                } else {
#pragma unroll
                for (int gg = 0; gg < 2; gg++) {
                    uint32_t qa[8], qb[8];
                    float da, db;
                    if (half == 0) {
                        if (gg == 0) tc8::split_blocks<0>(rrow, qa, qb, da, db);
                        else tc8::split_blocks<1>(rrow, qa, qb, da, db);
                    } else {
                        if (gg == 0) tc8::split_blocks<2>(rrow, qa, qb, da, db);
                        else tc8::split_blocks<3>(rrow, qa, qb, da, db);
                    }
                    const int blk = (half * 2 + gg) * 2;
                    uint32_t h[16];
                    uint32_t dd = (uint32_t)__half_as_ushort(__float2half_rn(da));   // the block's own f16 scale, back from f32 unchanged
                    dd |= dd << 16;
#pragma unroll
                    for (int j = 0; j < 8; j++) codes_to_f16(qa[j], dd, h[2 * j], h[2 * j + 1]);
                    tmem_st16(a_lane + (uint32_t)(slot * 128 + blk * 16), h);
                    dd = (uint32_t)__half_as_ushort(__float2half_rn(db));
                    dd |= dd << 16;
#pragma unroll
                    for (int j = 0; j < 8; j++) codes_to_f16(qb[j], dd, h[2 * j], h[2 * j + 1]);
                    tmem_st16(a_lane + (uint32_t)(slot * 128 + (blk + 1) * 16), h);
                }
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bar_aready[slot]);
                    mbar_arrive(&bar_rawfree[rs]);
                }
            }
        }
    } else if (warp >= tc8f::EPI_WARP0) {
        // ---- draining warps: lane quadrant warp % 4, column half (warp - tc8f::EPI_WARP0) / 4; once per tile
        const int q = warp & 3, ch = (warp - tc8f::EPI_WARP0) >> 2;
        const int row_in_tile = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + tc8f::ACC_COL0 + ((uint32_t)(q * 32) << 16) + (uint32_t)(ch * 128);
        uint32_t it = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, it++) {
            const int row_tile = t % p.row_tiles, col_tile = t / p.row_tiles;
            mbar_wait_nap(&bar_accfull, it & 1, fail, 128);
            tc_fence_after();
            const int64_t row = (int64_t)row_tile * ROWS + row_in_tile;
            const int col0 = col_tile * tc8f::NW + ch * 128;
            float *o = p.out + (size_t)col0 * p.ldy + row;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(lane_addr + (uint32_t)(c * 32), v);
                tmem_ld_wait();
                if (c == 3) {   // everything of this warp's part is in registers: the accumulator may be overwritten
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_accfree);
                }
                if (row < p.M) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (col0 + c * 32 + j < p.N) o[(size_t)(c * 32 + j) * p.ldy] = __uint_as_float(v[j]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && s_fail) atomicExch(p.err, 2);
}

static size_t tc8f_smem() { return (size_t)tc8f::B_STAGES * tc8f::B_STAGE + (size_t)tc8f::RAW_STAGES * tc8::RAW_BYTES + 1024; }   // the larger raw stage (Q8_0)

// The folded-scale GEMM for either weight format (the Q4_K planner and launcher in k_mmq_tc.cu call it for more than 64 columns)
uint64_t mm_fold_blob_unit() { return (uint64_t)4 * tc8f::B_STAGE; }
cudaError_t tc_encode_2d(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes, uint32_t box_rows,
                         uint32_t elem_bytes);
cudaError_t launch_mm_fold_f16(bool q4k, const void *W, int64_t K, int64_t M, int64_t N, const void *blobs, float *y, int64_t ldy, int *err,
                               cudaStream_t st) {
    CUtensorMap map;
    cudaError_t e = q4k ? tc_encode_2d(&map, W, (uint64_t)(K / 256 * 144), (uint64_t)M, 144, tc8::ROWS, 2)
                        : tc_encode_2d(&map, W, (uint64_t)(K / 32 * 34), (uint64_t)M, tc8::ROW_CHUNK, tc8::ROWS, 2);
    if (e != cudaSuccess) return e;
    static int sm_of[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!sm_of[dev]) cudaDeviceGetAttribute(&sm_of[dev], cudaDevAttrMultiProcessorCount, dev);
    Tc8fParams p{};
    p.act = (const uint8_t *)blobs;
    p.out = y;
    p.M = M;
    p.ldy = ldy;
    p.N = (int)N;
    p.nst = (int)(K / 256);
    p.row_tiles = (int)((M + tc8::ROWS - 1) / tc8::ROWS);
    p.col_tiles = (int)((N + tc8f::NW - 1) / tc8f::NW);
    p.err = err;
    const int tiles = p.row_tiles * p.col_tiles;
    const dim3 grid((unsigned)std::min(tiles, sm_of[dev]));
    return q4k ? launch_pdl(k_mm_q80_f16<true>, grid, dim3(tc8f::THREADS), tc8f_smem(), st, map, p)
               : launch_pdl(k_mm_q80_f16<false>, grid, dim3(tc8f::THREADS), tc8f_smem(), st, map, p);
}
cudaError_t launch_act_pack_fold(const ActLayout &a, const void *act, void *blobs, cudaStream_t st) {
    const char *ab = (const char *)act;
    k_act_pack_q80_f16<<<dim3((unsigned)(a.K / tc8f::KS), (unsigned)((a.N + tc8f::NW - 1) / tc8f::NW)), 256, 0, st>>>(
        (const int8_t *)(ab + a.qs_off), (const float *)(ab + a.d_off), a.K, (int)a.N, a.kind == ACT_Q8_K ? 256 : 32, (uint8_t *)blobs);
    return cudaGetLastError();
}

static size_t tc8w_smem() {
    return (size_t)tc8w::RAW_STAGES * tc8::RAW_BYTES + (size_t)tc8w::ACT_STAGES * tc8w::BLOB + (size_t)tc8w::A_RING * 8 * tc8::ROWS * sizeof(float) + 1024;
}

// ---------------------------------------------------------------- host side
template <int NPAD, int RS, int AS>
static size_t tc8_smem() {
    return (size_t)RS * tc8::RAW_BYTES + (size_t)AS * tc8_blob_bytes(NPAD) + (size_t)tc8::A_RING * 8 * tc8::ROWS * sizeof(float) + 1024;
}

void mmq_tc8_configure() {
    cudaFuncSetAttribute(k_mmq_tc_q80<16, 4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc8_smem<16, 4, 4>());
    cudaFuncSetAttribute(k_mmq_tc_q80<32, 4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc8_smem<32, 4, 4>());
    cudaFuncSetAttribute(k_mmq_tc_q80_wide, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc8w_smem());
    cudaFuncSetAttribute(k_mm_q80_f16<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc8f_smem());
    cudaFuncSetAttribute(k_mm_q80_f16<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc8f_smem());
}

bool mmq_tc8_supported(int64_t K, int64_t M, int64_t N) {
    return K % 256 == 0 && K >= 256 && M >= 1 && N > 4 && N <= (int64_t)tc8w::NW * 65535;   // column tiles are grid.y
}

TcPlan mmq_tc8_plan(int64_t K, int64_t M, int64_t N, int sm_count) {
    TcPlan t;
    t.nsb = (int)(K / 256);
    if (N > 64 && !getenv("TLB_NO_WIDE_TC") && !getenv("TLB_PROMPT_EXACT")) {
        // prompt-sized batches: 128 x 256 tiles, scales folded into f16 operands, one accumulator (k_mm_q80_f16)
        t.npad = tc8f::NW;
        t.n_split = 1;
        t.sb_per_split = t.nsb;
        t.streamk = 0;
        t.n_col_chunks = (int)((N + t.npad - 1) / t.npad);
        t.blob_unit = (uint64_t)4 * tc8f::B_STAGE;   // one unit of 256 elements of K = four stages of 64
        t.blob_bytes = (uint64_t)t.n_col_chunks * t.nsb * t.blob_unit;
        t.partial_bytes = 0;
        return t;
    }
    if (N > 64 && !getenv("TLB_NO_WIDE_TC")) {
        // the same batches with the reference's integer arithmetic (TLB_PROMPT_EXACT=1): 128-column tiles, whole K per
        // CTA (k_mmq_tc_q80_wide), row tiles x column tiles fill the GPU
        t.npad = tc8w::NW;
        t.n_split = 1;
        t.sb_per_split = t.nsb;
        t.streamk = 0;
        t.n_col_chunks = (int)((N + t.npad - 1) / t.npad);
        t.blob_unit = (uint64_t)tc8_blob_bytes(t.npad);
        t.blob_bytes = (uint64_t)t.n_col_chunks * t.nsb * t.blob_unit;
        t.partial_bytes = 0;
        return t;
    }
    t.npad = N <= 16 ? 16 : 32;
    const int64_t tiles = (M + tc8::ROWS - 1) / tc8::ROWS;
    // same model as the Q4_K kernel, with this kernel's time per stage
    int best = 1;
    double best_score = 1e30;
    for (int s = 1; s <= t.nsb && s <= 16; s++) {
        const int per = (t.nsb + s - 1) / s;
        if (s > 1 && per < 2) break;
        const int splits = (t.nsb + per - 1) / per;
        if (splits != s) continue;
        const int64_t waves = (tiles * splits + sm_count - 1) / sm_count;
        const double score = (double)waves * (2.3 + 1.0 * per) + (splits > 1 ? 2.0 : 0.0);
        if (score < best_score) { best_score = score; best = splits; }
    }
    t.n_split = best;
    t.sb_per_split = (t.nsb + best - 1) / best;
    t.streamk = 0;
    t.n_col_chunks = (int)((N + t.npad - 1) / t.npad);
    t.blob_unit = (uint64_t)tc8_blob_bytes(t.npad);
    t.blob_bytes = (uint64_t)t.n_col_chunks * t.nsb * t.blob_unit;
    t.partial_bytes = best > 1 ? (uint64_t)best * std::min<int64_t>(N, t.npad) * M * 4 : 0;
    return t;
}

cudaError_t launch_act_pack_tc8(const ActLayout &a, const void *act, int npad, void *blobs, cudaStream_t st) {
    const char *ab = (const char *)act;
    if (npad == tc8f::NW) {
        k_act_pack_q80_f16<<<dim3((unsigned)(a.K / tc8f::KS), (unsigned)((a.N + npad - 1) / npad)), 256, 0, st>>>(
            (const int8_t *)(ab + a.qs_off), (const float *)(ab + a.d_off), a.K, (int)a.N, a.kind == ACT_Q8_K ? 256 : 32, (uint8_t *)blobs);
        return cudaGetLastError();
    }
    k_act_pack_q80<<<dim3((unsigned)(a.K / 256), (unsigned)((a.N + npad - 1) / npad)), 256, 0, st>>>((const int8_t *)(ab + a.qs_off), (const float *)(ab + a.d_off), a.K, (int)a.N, npad,
                                                         (uint8_t *)blobs);
    return cudaGetLastError();
}

cudaError_t tc_encode_2d(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes, uint32_t box_rows,
                         uint32_t elem_bytes);
void launch_mmq_reduce(const float *partial, float *y, int64_t total, int n_split, cudaStream_t st);

cudaError_t launch_mmq_tc8(const TcPlan &t, const void *W, int64_t K, int64_t M, int64_t N, const void *blobs, float *y, int64_t ldy,
                           void *partial, int *err, cudaStream_t st) {
    CUtensorMap map;
    // described in 16-bit elements: a 272-byte box is 136 of them (the limit is 256 elements per dimension)
    cudaError_t e = tc_encode_2d(&map, W, (uint64_t)(K / 32 * 34), (uint64_t)M, tc8::ROW_CHUNK, tc8::ROWS, 2);
    if (e != cudaSuccess) return e;
    if (t.npad == tc8f::NW) return launch_mm_fold_f16(false, W, K, M, N, blobs, y, ldy, err, st);
    if (t.npad == tc8w::NW) {
        Tc8Params p{};
        p.act = (const uint8_t *)blobs;
        p.out = y;
        p.M = M;
        p.N = (int)N;
        p.npad = t.npad;
        p.nst = p.st_per_split = t.nsb;
        p.n_split = 1;
        p.ldy = ldy;
        p.err = err;
        return launch_pdl(k_mmq_tc_q80_wide, dim3((unsigned)((M + tc8::ROWS - 1) / tc8::ROWS), (unsigned)t.n_col_chunks), dim3(tc8w::THREADS),
                          tc8w_smem(), st, map, p);
    }
    dim3 grid((unsigned)((M + tc8::ROWS - 1) / tc8::ROWS), (unsigned)t.n_split);
    for (int c = 0; c < t.n_col_chunks; c++) {   // one launch per chunk of npad columns
        const int64_t n0 = (int64_t)c * t.npad, nc = std::min<int64_t>(t.npad, N - n0);
        Tc8Params p;
        p.act = (const uint8_t *)blobs + (size_t)c * t.nsb * t.blob_unit;
        p.M = M;
        p.N = (int)nc;
        p.npad = t.npad;
        p.nst = t.nsb;
        p.st_per_split = t.sb_per_split;
        p.n_split = t.n_split;
        p.err = err;
        float *yc = y + n0 * ldy;
        if (t.n_split > 1) {
            p.out = (float *)partial;
            p.ldy = M;
        } else {
            p.out = yc;
            p.ldy = ldy;
        }
        if (t.npad == 16) e = launch_pdl(k_mmq_tc_q80<16, 4, 4>, grid, dim3(tc8::THREADS), tc8_smem<16, 4, 4>(), st, map, p);
        else e = launch_pdl(k_mmq_tc_q80<32, 4, 4>, grid, dim3(tc8::THREADS), tc8_smem<32, 4, 4>(), st, map, p);
        if (e != cudaSuccess) return e;
        if (t.n_split > 1) {
            if (ldy != M) return cudaErrorInvalidValue;
            launch_mmq_reduce((const float *)partial, yc, nc * M, t.n_split, st);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

}  // namespace tlb
