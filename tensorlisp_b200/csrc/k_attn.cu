// Paged-attention decode and its cache write (reference: the CUSTOM nodes lowered by
// crates/kernels/src/cuda/lower.rs:660-759 onto the vendored vLLM kernels in
// crates/kernels/src/cuda/shaders/, launcher maths in cuda/paged_attn.rs).
//
// The KV pools are only ever written by the cache-write node and read by the attention node
// (scheme/core.ss:218-220), so their layout is the executor's own: f16
// [block][kv_head][slot][head_size] for keys and for values -- every (block, kv_head) page is one
// contiguous run of block_size rows, and a row is head_size*2 bytes.
//
// k_paged_attn: grid (context chunk, kv head x query-head group, sequence). A CTA serves ALL query
// heads that share one KV head (GQA), so each K/V byte is read from HBM once. Each warp streams
// 16-token tiles of K and V through its own cp.async ring in shared memory (XOR-swizzled rows,
// conflict-free ldmatrix), computes S = Q K^T and O += P V on the f16 tensor cores
// (mma.sync.m16n8k16, f32 accumulate; the query heads of the group are the M rows) with an online
// softmax in base 2, and the warps' (max, sum, O) are merged at the end. With more than one chunk the
// CTA writes an f32 partial (max, sum, O) and k_paged_reduce merges the chunks (split-K).
#include <algorithm>
#include <cstdlib>
#include <climits>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kernels.h"
#include "pdl.cuh"
#include "rowquant.cuh"
#include "tlb_internal.h"

namespace tlb {

constexpr int PA_WARPS = 4;
constexpr int PA_STAGES = 3;
constexpr int PA_TILE = 16;  // tokens per tile

__device__ __forceinline__ uint32_t s_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

struct PagedParams {
    const __half *q;       // [seqs][heads][HS]
    const __half *kpool;   // [block][kv_heads][block_size][HS]
    const __half *vpool;
    const int32_t *tables; // [seqs][max_blocks]
    const int32_t *lens;   // [seqs]
    __half *out;           // [seqs][heads][HS]
    float *partial;        // [seqs][heads][n_chunks][HS + 2]  (max, sum, O) when n_chunks > 1
    int heads, kv_heads, group, groups_per_kv, block_size, block_shift, max_blocks, chunk_tokens, n_chunks;
    int hs;                // head size (the tensor-core kernel has it as a template argument)
    int ctx_cap;           // min(maximum context, max_blocks * block_size): no length from the caller reaches past a table row
    uint32_t pool_blocks;  // pages in each pool; 0x80000000 when this launch does not know (block ids are then only checked for sign)
    int *err;              // device error word, or null: set to TLB_ERR_INDEX when a length or a block id was out of range
    float scale_log2;      // softmax scale * log2(e)
    // fuse_rq: the f16 output row is also quantized to Q8_K (and packed for the tensor-core mul_mat) right here, as the
    // row quantizer in RQ_F16 mode would do in a launch of its own; only without a context split (n_chunks == 1)
    int fuse_rq;
    RowQuantArgs rq;
};
// A context length beyond the cap is cut to the cap; a CTA that meets a block id outside the pools leaves without
// touching them; either way the error word tells the host that the result is not to be used.
__device__ __forceinline__ int paged_ctx(const PagedParams &p, int seq) {
    const int n = p.lens[seq];
    if (n < 0 || n > p.ctx_cap) {
        if (p.err) atomicExch(p.err, TLB_ERR_INDEX);
        return n < 0 ? 0 : p.ctx_cap;
    }
    return n;
}

template <int HS>
__global__ void __launch_bounds__(PA_WARPS * 32) k_paged_attn(PagedParams p) {
    griddep_launch();
    griddep_wait();   // the pools and the query were written by the kernel before this one
    constexpr int ROW_BYTES = HS * 2;
    constexpr int CHUNKS = ROW_BYTES / 16;             // 16-byte chunks per row
    constexpr int TILE_BYTES = PA_TILE * ROW_BYTES;    // one of K / V
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int KS = HS / 16;                        // k-steps of Q K^T
    constexpr int ND = HS / 8;                         // n-tiles of P V
    extern __shared__ __align__(128) uint8_t smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int chunk = blockIdx.x, seq = blockIdx.z;
    const int kvh = blockIdx.y / p.groups_per_kv, grp = blockIdx.y % p.groups_per_kv;
    const int ctx = paged_ctx(p, seq);
    const int c_begin = chunk * p.chunk_tokens;
    if (c_begin >= ctx && !(chunk == 0)) return;  // nothing to do; the reduce skips this chunk
    const int c_end = min(ctx, c_begin + p.chunk_tokens);
    const int head0 = kvh * p.group + grp * 16;               // first query head of this CTA
    const int nrows = min(16, p.group - grp * 16);            // query heads served here
    const int n_tiles = c_end > c_begin ? (c_end - c_begin + PA_TILE - 1) / PA_TILE : 0;
    const int32_t *table = p.tables + (size_t)seq * p.max_blocks;
    {
        // The block ids of this CTA's stretch of the context are checked here, once, and not in the copy loop below
        // (every instruction there is paid per 16 bytes moved): an id outside the pools never becomes an address,
        // the CTA reports it and leaves, and its part of the result stays unwritten.
        bool bad = false;
        if (c_end > c_begin)
            for (int b = (c_begin >> p.block_shift) + (int)threadIdx.x; b <= ((c_end - 1) >> p.block_shift); b += PA_WARPS * 32)
                bad |= (uint32_t)table[b] >= p.pool_blocks;   // negative ids are large here
        if (__syncthreads_or(bad)) {
            if (threadIdx.x == 0 && p.err) atomicExch(p.err, TLB_ERR_INDEX);
            return;
        }
    }

    // ---- Q fragments (A operand, rows = query heads of the group, zero beyond nrows)
    uint32_t qa[KS][4];
    {
        const __half *q0 = p.q + ((size_t)seq * p.heads + head0) * HS;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const int c0 = ks * 16 + 2 * t;
            qa[ks][0] = g < nrows ? *reinterpret_cast<const uint32_t *>(q0 + (size_t)g * HS + c0) : 0u;
            qa[ks][1] = g + 8 < nrows ? *reinterpret_cast<const uint32_t *>(q0 + (size_t)(g + 8) * HS + c0) : 0u;
            qa[ks][2] = g < nrows ? *reinterpret_cast<const uint32_t *>(q0 + (size_t)g * HS + c0 + 8) : 0u;
            qa[ks][3] = g + 8 < nrows ? *reinterpret_cast<const uint32_t *>(q0 + (size_t)(g + 8) * HS + c0 + 8) : 0u;
        }
    }

    uint8_t *ring = smem + (size_t)warp * PA_STAGES * STAGE_BYTES;
    const size_t page_stride = (size_t)p.block_size * HS;  // elements per (block, kv_head)

    // issue the cp.asyncs of this warp's tile `i` (tile index within the warp's sequence)
    auto issue = [&](int i) {
        const int tile = warp + i * PA_WARPS;
        if (tile < n_tiles) {
            uint8_t *st = ring + (size_t)(i % PA_STAGES) * STAGE_BYTES;
            const int tok0 = c_begin + tile * PA_TILE;
            // K and V rows of a token sit at the same offset of their pools, and the rows of a page follow one
            // another there. With pages of 8 tokens or more (block sizes are powers of two) the tile's first 8
            // tokens lie in one page and its last 8 in one page: two table lookups and two base addresses per tile, so that every
            // 16-byte copy below costs an add and little else (each instruction here is paid per 16 bytes moved).
            constexpr int ROWS_PER_IT = 32 / CHUNKS, N_IT = PA_TILE / ROWS_PER_IT;
            static_assert(N_IT % 2 == 0 && 8 % ROWS_PER_IT == 0, "a copy step stays inside one half of the tile");
            const int col = lane % CHUNKS, row0 = lane / CHUNKS;
            const int n_live = c_end - tok0;   // >= 1: rows at and past it are zero-filled
            const uint32_t dst0 = s_u32(st);
            if (p.block_shift < 3) {
                // pages of fewer than 8 tokens: a lookup and an address per row
#pragma unroll
                for (int it = 0; it < N_IT; it++) {
                    const int row = it * ROWS_PER_IT + row0;
                    const int tok = tok0 + row;
                    const bool live = row < n_live;
                    size_t off = 0;
                    if (live) {
                        const int blk = table[tok >> p.block_shift];
                        off = ((size_t)blk * p.kv_heads + kvh) * page_stride + (size_t)(tok & (p.block_size - 1)) * HS + col * 8;
                    }
                    const uint32_t dst = dst0 + row * ROW_BYTES + ((col ^ (row & 7)) * 16);
                    cp_async16(dst, p.kpool + off, live ? 16 : 0);
                    cp_async16(dst + TILE_BYTES, p.vpool + off, live ? 16 : 0);
                }
                cp_commit();
                return;
            }
            size_t off_half[2];
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const int tok = tok0 + 8 * hf;
                const int blk = tok < c_end ? table[tok >> p.block_shift] : 0;
                off_half[hf] = ((size_t)blk * p.kv_heads + kvh) * page_stride + (size_t)((tok & (p.block_size - 1)) + row0) * HS + col * 8;
            }
#pragma unroll
            for (int it = 0; it < N_IT; it++) {
                constexpr int HALF_IT = N_IT / 2;
                const int row = it * ROWS_PER_IT + row0;
                const bool live = row < n_live;
                const size_t off = live ? off_half[it / HALF_IT] + (size_t)((it % HALF_IT) * ROWS_PER_IT) * HS : 0;
                const uint32_t dst = dst0 + row * ROW_BYTES + ((col ^ (row & 7)) * 16);
                cp_async16(dst, p.kpool + off, live ? 16 : 0);   // rows past the context are zero-filled
                cp_async16(dst + TILE_BYTES, p.vpool + off, live ? 16 : 0);
            }
        }
        cp_commit();
    };

    float o[ND][4];
#pragma unroll
    for (int n = 0; n < ND; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};

    const int my_tiles = n_tiles > warp ? (n_tiles - warp + PA_WARPS - 1) / PA_WARPS : 0;
#pragma unroll
    for (int i = 0; i < PA_STAGES - 1; i++) issue(i);

    for (int i = 0; i < my_tiles; i++) {
        issue(i + PA_STAGES - 1);
        cp_wait<PA_STAGES - 1>();
        __syncwarp();
        const uint8_t *st = ring + (size_t)(i % PA_STAGES) * STAGE_BYTES;
        const uint32_t kbase = s_u32(st), vbase = kbase + TILE_BYTES;
        const int tok0 = c_begin + (warp + i * PA_WARPS) * PA_TILE;

        // ---- S = Q K^T for 16 tokens (two n-tiles of 8)
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const int mi = lane >> 3, r = lane & 7;
            const int row = (mi >> 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const int col = ks * 2 + (mi & 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4(kbase + row * ROW_BYTES + ((col ^ (row & 7)) * 16), b0, b1, b2, b3);
                mma16816(s[0], qa[ks], b0, b1);
                mma16816(s[1], qa[ks], b2, b3);
            }
        }
        // ---- online softmax (base 2); rows g and g+8
        float rmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] *= p.scale_log2;
        if (tok0 + PA_TILE > c_end) {   // only the last tile of a context has tokens to mask
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (tok0 + j * 8 + 2 * t + (e & 1) >= c_end) s[j][e] = -CUDART_INF_F;
        }
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) rmax[e >> 1] = fmaxf(rmax[e >> 1], s[j][e]);
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
            rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
            const float m_new = fmaxf(m_run[h], rmax[h]);
            m_use[h] = m_new == -CUDART_INF_F ? 0.f : m_new;
            corr[h] = exp2f(m_run[h] - m_use[h]);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
        // P as two f16 terms (value and rounding residual): the product with V is then accurate to
        // ~2^-22, which matters because the next MUL_MAT re-quantizes this output to int8
        uint32_t pa[4], pr[4];
        {
            float pv[2][4], rs[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    pv[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
                    l_run[e >> 1] += pv[j][e];
                    rs[j][e] = pv[j][e] - __half2float(__float2half_rn(pv[j][e]));
                }
            pa[0] = pack_h2(pv[0][0], pv[0][1]);
            pa[1] = pack_h2(pv[0][2], pv[0][3]);
            pa[2] = pack_h2(pv[1][0], pv[1][1]);
            pa[3] = pack_h2(pv[1][2], pv[1][3]);
            pr[0] = pack_h2(rs[0][0], rs[0][1]);
            pr[1] = pack_h2(rs[0][2], rs[0][3]);
            pr[2] = pack_h2(rs[1][0], rs[1][1]);
            pr[3] = pack_h2(rs[1][2], rs[1][3]);
        }
        // ---- O = O * corr + P V. Once the running maxima have settled, corr is exactly 1 for every row of the
        // warp in most tiles: the multiplications are then left out (a product with 1.0f changes no bit).
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
            for (int nd = 0; nd < ND; nd++) {
                o[nd][0] *= corr[0]; o[nd][1] *= corr[0]; o[nd][2] *= corr[1]; o[nd][3] *= corr[1];
            }
        }
        {
            const int mi = lane >> 3, r = lane & 7;
            const int row = (mi & 1) * 8 + r;
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {
                const int col = nd + (mi >> 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(vbase + row * ROW_BYTES + ((col ^ (row & 7)) * 16), b0, b1, b2, b3);
                mma16816(o[nd], pa, b0, b1);
                mma16816(o[nd], pr, b0, b1);
                mma16816(o[nd + 1], pa, b2, b3);
                mma16816(o[nd + 1], pr, b2, b3);
            }
        }
    }
    cp_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();  // every warp's ring is drained: shared memory is reused for the merge

    // ---- merge the warps: ml[w][row] = (m, l), acc[w][row][HS]
    float *ml = reinterpret_cast<float *>(smem);                   // [PA_WARPS][16][2]
    float *acc = ml + PA_WARPS * 16 * 2;                           // [PA_WARPS][16][HS]
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int row = g + 8 * h;
        if (row < nrows) {
            if (t == 0) {
                ml[(warp * 16 + row) * 2] = m_run[h];
                ml[(warp * 16 + row) * 2 + 1] = l_run[h];
            }
#pragma unroll
            for (int nd = 0; nd < ND; nd++) {
                float2 v = make_float2(o[nd][2 * h], o[nd][2 * h + 1]);
                *reinterpret_cast<float2 *>(&acc[((size_t)warp * 16 + row) * HS + nd * 8 + 2 * t]) = v;
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nrows * HS; idx += PA_WARPS * 32) {
        const int row = idx / HS, d = idx % HS;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < PA_WARPS; w++) m = fmaxf(m, ml[(w * 16 + row) * 2]);
        const float mu = m == -CUDART_INF_F ? 0.f : m;
        float l = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < PA_WARPS; w++) {
            const float f = exp2f(ml[(w * 16 + row) * 2] - mu);
            l += ml[(w * 16 + row) * 2 + 1] * f;
            a += acc[((size_t)w * 16 + row) * HS + d] * f;
        }
        const int head = head0 + row;
        if (p.n_chunks == 1) {
            const __half o16 = __float2half_rn(l > 0.f ? a / l : 0.f);
            p.out[((size_t)seq * p.heads + head) * HS + d] = o16;
            if (p.fuse_rq) acc[(size_t)PA_WARPS * 16 * HS + idx] = __half2float(o16);   // behind the warps' partial outputs
        } else {
            float *pp = p.partial + (((size_t)seq * p.heads + head) * p.n_chunks + chunk) * (HS + 2);
            pp[2 + d] = a;
            if (d == 0) { pp[0] = m; pp[1] = l; }
        }
    }
    if (p.fuse_rq && p.n_chunks == 1) {
        // the CTA's heads are nrows * HS consecutive elements of the token's row: whole 256-value Q8_K blocks, one per warp
        __syncthreads();
        const float *rowv = acc + (size_t)PA_WARPS * 16 * HS;
        const int nblk = (int)(p.rq.K / 256), blk0 = head0 * HS / 256;
        for (int w = warp; w < nrows * HS / 256; w += PA_WARPS) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = rowv[w * 256 + lane * 8 + e];
            rq_quant_block(p.rq, seq, blk0 + w, nblk, lane, v);
        }
    }
}

template <int HS>
__global__ void __launch_bounds__(128) k_paged_reduce(PagedParams p) {
    griddep_launch();
    griddep_wait();
    const int head = blockIdx.x, seq = blockIdx.y;
    const int ctx = paged_ctx(p, seq);
    const int valid = ctx > 0 ? min(p.n_chunks, (ctx + p.chunk_tokens - 1) / p.chunk_tokens) : 0;
    const float *pp = p.partial + ((size_t)seq * p.heads + head) * p.n_chunks * (HS + 2);
    float m = -CUDART_INF_F;
    for (int c = 0; c < valid; c++) m = fmaxf(m, pp[(size_t)c * (HS + 2)]);
    const float mu = m == -CUDART_INF_F ? 0.f : m;
    for (int d = threadIdx.x; d < HS; d += blockDim.x) {
        float l = 0.f, a = 0.f;
        for (int c = 0; c < valid; c++) {
            const float f = exp2f(pp[(size_t)c * (HS + 2)] - mu);
            l += pp[(size_t)c * (HS + 2) + 1] * f;
            a += pp[(size_t)c * (HS + 2) + 2 + d] * f;
        }
        p.out[((size_t)seq * p.heads + head) * HS + d] = __float2half_rn(l > 0.f ? a / l : 0.f);
    }
}

// ---------------------------------------------------------------- any other head size
// The head sizes of the reference's list (crates/kernels/src/cuda/paged_attn.rs:24: 64 80 96 112 128 192 256 512) that
// the tensor-core kernel above does not take, and any other multiple of 8 up to 512: one CTA per (sequence, query
// head), a warp per token in turn, a lane per 16-byte chunk of the row (C chunks per lane), f32 dot product, online
// softmax and accumulation per warp, the warps merged through shared memory. No context split. Not a tuned kernel:
// a query head re-reads its KV head's pages (from L2 within a group).
template <int C>
__global__ void __launch_bounds__(PA_WARPS * 32) k_paged_attn_any(PagedParams p) {
    griddep_launch();
    griddep_wait();
    __shared__ float ml[PA_WARPS][2];
    __shared__ float accs[PA_WARPS][512];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y, seq = blockIdx.z, kvh = head / p.group;
    const int hs = p.hs, chunks = hs >> 3;
    const int ctx = paged_ctx(p, seq);
    const int32_t *table = p.tables + (size_t)seq * p.max_blocks;
    {
        bool bad = false;
        if (ctx > 0)
            for (int b = (int)threadIdx.x; b <= ((ctx - 1) >> p.block_shift); b += PA_WARPS * 32)
                bad |= (uint32_t)table[b] >= p.pool_blocks;
        if (__syncthreads_or(bad)) {
            if (threadIdx.x == 0 && p.err) atomicExch(p.err, TLB_ERR_INDEX);
            return;
        }
    }
    float qf[C][8], acc[C][8];
    const __half *q0 = p.q + ((size_t)seq * p.heads + head) * hs;
#pragma unroll
    for (int c = 0; c < C; c++) {
        const int ch = lane + 32 * c;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (ch < chunks) raw = *reinterpret_cast<const uint4 *>(q0 + ch * 8);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float2 f = __half22float2(h[e]);
            qf[c][2 * e] = f.x;
            qf[c][2 * e + 1] = f.y;
            acc[c][2 * e] = acc[c][2 * e + 1] = 0.f;
        }
    }
    float m_run = -CUDART_INF_F, l_run = 0.f;
    const size_t page_stride = (size_t)p.block_size * hs;
    for (int tok = warp; tok < ctx; tok += PA_WARPS) {
        const int blk = table[tok >> p.block_shift];
        const size_t off = ((size_t)blk * p.kv_heads + kvh) * page_stride + (size_t)(tok & (p.block_size - 1)) * hs;
        uint4 vraw[C];
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < C; c++) {
            const int ch = lane + 32 * c;
            uint4 kraw = make_uint4(0, 0, 0, 0);
            vraw[c] = make_uint4(0, 0, 0, 0);
            if (ch < chunks) {
                kraw = *reinterpret_cast<const uint4 *>(p.kpool + off + ch * 8);
                vraw[c] = *reinterpret_cast<const uint4 *>(p.vpool + off + ch * 8);
            }
            const __half2 *h = reinterpret_cast<const __half2 *>(&kraw);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = __half22float2(h[e]);
                dot = fmaf(qf[c][2 * e], f.x, dot);
                dot = fmaf(qf[c][2 * e + 1], f.y, dot);
            }
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sh);
        const float sc = dot * p.scale_log2;
        const float m_new = fmaxf(m_run, sc);
        const float corr = exp2f(m_run - m_new), pw = exp2f(sc - m_new);
        m_run = m_new;
        l_run = l_run * corr + pw;
#pragma unroll
        for (int c = 0; c < C; c++) {
            const __half2 *h = reinterpret_cast<const __half2 *>(&vraw[c]);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = __half22float2(h[e]);
                acc[c][2 * e] = fmaf(pw, f.x, acc[c][2 * e] * corr);
                acc[c][2 * e + 1] = fmaf(pw, f.y, acc[c][2 * e + 1] * corr);
            }
        }
    }
    if (lane == 0) {
        ml[warp][0] = m_run;
        ml[warp][1] = l_run;
    }
#pragma unroll
    for (int c = 0; c < C; c++) {
        const int ch = lane + 32 * c;
        if (ch < chunks) {
#pragma unroll
            for (int e = 0; e < 8; e++) accs[warp][ch * 8 + e] = acc[c][e];
        }
    }
    __syncthreads();
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < PA_WARPS; w++) m = fmaxf(m, ml[w][0]);
    const float mu = m == -CUDART_INF_F ? 0.f : m;
    for (int d = threadIdx.x; d < hs; d += PA_WARPS * 32) {
        float l = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < PA_WARPS; w++) {
            const float f = exp2f(ml[w][0] - mu);
            l += ml[w][1] * f;
            a += accs[w][d] * f;
        }
        p.out[((size_t)seq * p.heads + head) * hs + d] = __float2half_rn(l > 0.f ? a / l : 0.f);
    }
}

// ---------------------------------------------------------------- host side
// the heads of a CTA make whole 256-value blocks of the output row, at a block boundary
bool paged_quant_fusable(const PagedGeom &g) {
    const int group = g.heads / g.kv_heads;
    return (g.hs == 128 && group % 2 == 0 && (group <= 16 || group % 16 == 0)) || (g.hs == 256 && (group <= 16 || group % 16 == 0));
}

static size_t pa_smem(int hs) {
    const size_t ring = (size_t)PA_WARPS * PA_STAGES * 2 * PA_TILE * hs * 2;
    const size_t merge = (size_t)PA_WARPS * 16 * (2 + hs) * 4 + (size_t)16 * hs * 4;   // + the output row of the fused quantizer
    return ring > merge ? ring : merge;
}

void attn_configure() {
    cudaFuncSetAttribute(k_paged_attn<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pa_smem(64));
    cudaFuncSetAttribute(k_paged_attn<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pa_smem(128));
    cudaFuncSetAttribute(k_paged_attn<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pa_smem(256));
}

static bool pa_tensor_core_hs(int hs) { return hs == 64 || hs == 128 || hs == 256; }

bool paged_supported(const PagedGeom &g) {
    if (g.hs < 8 || g.hs > 512 || g.hs % 8 != 0) return false;
    if (g.kv_heads < 1 || g.heads % g.kv_heads != 0) return false;
    if (g.block_size < 1 || g.max_blocks < 1 || (g.block_size & (g.block_size - 1)) != 0) return false;
    return true;
}

// Context chunk per CTA. Measured on B200 (32 sequences x 8 kv heads x 2048 tokens, chunk swept from 128
// to 2048 tokens): time = waves x (0.024 us per token + 2.6 us per CTA) + 2.5 us for the reduce launch
// when the context is split, where a wave is (SMs x resident CTAs) CTAs. So a CTA start costs as much
// as 110 tokens and splitting as much as 100: the context is split only as far as it takes to fill
// the machine, and the split count minimises that model.
void paged_plan(PagedGeom &g, int sm_count) {
    if (!pa_tensor_core_hs(g.hs)) {   // the kernel for the other head sizes takes a whole context per CTA
        g.chunk_tokens = (int)std::max<int64_t>(64, (g.max_ctx + 63) / 64 * 64);
        g.n_chunks = 1;
        return;
    }
    const int group = g.heads / g.kv_heads;
    const int64_t base = (int64_t)g.seqs * g.kv_heads * ((group + 15) / 16);
    const int64_t per_sm = std::max<int64_t>(1, std::min<int64_t>(3, (227 * 1024) / ((int64_t)pa_smem(g.hs) + 1024)));
    const int64_t slots = (int64_t)sm_count * per_sm;
    int64_t best_ct = 64, best_cost = INT64_MAX;
    for (int64_t n = 1; n <= 256; n++) {
        int64_t ct = ((g.max_ctx + n - 1) / n + 63) / 64 * 64;
        if (ct < 64) ct = 64;
        const int64_t nn = std::max<int64_t>(1, (g.max_ctx + ct - 1) / ct);
        const int64_t waves = (base * nn + slots - 1) / slots;
        const int64_t cost = waves * (ct + 110) + (nn > 1 ? 100 : 0);
        if (cost < best_cost) { best_cost = cost; best_ct = ct; }
        if (ct == 64) break;
    }
    if (const char *e = getenv("TLB_PA_CHUNK")) {   // tuning knob: chunk length in tokens (a multiple of 64)
        const int64_t v = atoll(e);
        if (v >= 64 && v % 64 == 0) best_ct = v;
    }
    g.chunk_tokens = (int)best_ct;
    g.n_chunks = (int)std::max<int64_t>(1, (g.max_ctx + best_ct - 1) / best_ct);
}

uint64_t paged_scratch_bytes(const PagedGeom &g) {
    if (g.n_chunks <= 1) return 0;
    return (uint64_t)g.seqs * g.heads * g.n_chunks * (g.hs + 2) * 4;
}

template <int HS>
static cudaError_t launch_pa(const PagedGeom &g, const PagedParams &p, cudaStream_t st) {
    dim3 grid((unsigned)g.n_chunks, (unsigned)(g.kv_heads * p.groups_per_kv), (unsigned)g.seqs);
    cudaError_t e = launch_pdl(k_paged_attn<HS>, grid, dim3(PA_WARPS * 32), pa_smem(HS), st, p);
    if (e == cudaSuccess && g.n_chunks > 1) e = launch_pdl(k_paged_reduce<HS>, dim3((unsigned)g.heads, (unsigned)g.seqs), dim3(128), 0, st, p);
    return e;
}

cudaError_t launch_paged_attention(const PagedGeom &g, const void *q, const void *kpool, const void *vpool,
                                   const int32_t *tables, const int32_t *lens, void *out, void *scratch,
                                   int64_t pool_blocks, int *err, cudaStream_t st, const RowQuantArgs *rq) {
    if (g.seqs == 0 || g.heads == 0) return cudaSuccess;
    PagedParams p;
    p.q = (const __half *)q;
    p.kpool = (const __half *)kpool;
    p.vpool = (const __half *)vpool;
    p.tables = tables;
    p.lens = lens;
    p.out = (__half *)out;
    p.partial = (float *)scratch;
    p.heads = g.heads;
    p.kv_heads = g.kv_heads;
    p.group = g.heads / g.kv_heads;
    p.groups_per_kv = (p.group + 15) / 16;
    p.block_size = g.block_size;
    p.block_shift = 0;
    while ((1 << p.block_shift) < g.block_size) p.block_shift++;
    p.max_blocks = g.max_blocks;
    p.chunk_tokens = g.chunk_tokens;
    p.n_chunks = g.n_chunks;
    p.hs = g.hs;
    p.ctx_cap = (int)std::min<int64_t>(g.max_ctx, (int64_t)g.max_blocks * g.block_size);
    p.pool_blocks = pool_blocks > 0 && pool_blocks < 0x80000000ll ? (uint32_t)pool_blocks : 0x80000000u;
    p.err = err;
    p.fuse_rq = 0;
    p.rq = RowQuantArgs{};
    if (rq) {
        if (g.n_chunks != 1 || !paged_quant_fusable(g)) return cudaErrorInvalidValue;
        p.fuse_rq = 1;
        p.rq = *rq;
    }
    p.scale_log2 = g.scale * 1.4426950408889634f;
    switch (g.hs) {
        case 64: return launch_pa<64>(g, p, st);
        case 128: return launch_pa<128>(g, p, st);
        case 256: return launch_pa<256>(g, p, st);
        default: break;
    }
    if (!paged_supported(g) || g.n_chunks != 1) return cudaErrorInvalidValue;
    const dim3 grid(1, (unsigned)g.heads, (unsigned)g.seqs);
    if (g.hs <= 256) return launch_pdl(k_paged_attn_any<1>, grid, dim3(PA_WARPS * 32), 0, st, p);
    return launch_pdl(k_paged_attn_any<2>, grid, dim3(PA_WARPS * 32), 0, st, p);
}

// cache write: key/value f16 [kv_heads*hs, tokens] -> pools at slot = block*block_size + offset
// (reshape_and_cache of the reference; a negative slot skips the token)
__global__ void k_cache_write(int kv_heads, int hs, int block_size, const uint4 *key, const uint4 *value, uint4 *kpool,
                              uint4 *vpool, const int64_t *slots, int64_t pool_slots, int *err) {
    const int tok = blockIdx.x;
    const int64_t slot = slots[tok];
    if (slot < 0) return;
    if (slot >= pool_slots) {   // beyond the pools: nothing is written, the host hears of it
        if (threadIdx.x == 0 && err) atomicExch(err, TLB_ERR_INDEX);
        return;
    }
    const int64_t blk = slot / block_size, off = slot % block_size;
    const int cpr = hs / 8;  // 16-byte chunks per head row
    for (int i = threadIdx.x; i < kv_heads * cpr; i += blockDim.x) {
        const int h = i / cpr, c = i % cpr;
        const size_t dst = (((size_t)blk * kv_heads + h) * block_size + off) * cpr + c;
        const size_t src = (size_t)tok * kv_heads * cpr + i;
        kpool[dst] = key[src];
        vpool[dst] = value[src];
    }
}
cudaError_t launch_cache_write(int tokens, int kv_heads, int hs, int block_size, const void *key, const void *value,
                               void *kpool, void *vpool, const int64_t *slots, int64_t pool_slots, int *err, cudaStream_t st) {
    if (tokens == 0) return cudaSuccess;
    k_cache_write<<<tokens, 128, 0, st>>>(kv_heads, hs, block_size, (const uint4 *)key, (const uint4 *)value, (uint4 *)kpool,
                                          (uint4 *)vpool, slots, pool_slots, err);
    return cudaGetLastError();
}

// pool -> dense [ctx, kv_heads, hs] per sequence (gather_kv_cache of the reference)
__global__ void k_paged_gather(int kv_heads, int hs, int block_size, int max_blocks, const uint4 *pool, const int32_t *tables,
                               const int32_t *lens, const int64_t *seq_offsets, uint4 *out) {
    const int seq = blockIdx.y, tok = blockIdx.x;
    if (tok >= lens[seq]) return;
    const int blk = tables[(size_t)seq * max_blocks + tok / block_size], off = tok % block_size;
    const int cpr = hs / 8;
    for (int i = threadIdx.x; i < kv_heads * cpr; i += blockDim.x) {
        const int h = i / cpr, c = i % cpr;
        out[(size_t)(seq_offsets[seq] + tok) * kv_heads * cpr + i] = pool[(((size_t)blk * kv_heads + h) * block_size + off) * cpr + c];
    }
}
cudaError_t launch_paged_gather(int seqs, int kv_heads, int hs, int block_size, int max_blocks, const void *pool,
                                const int32_t *tables, const int32_t *lens, const int64_t *seq_offsets, void *out,
                                int max_ctx, cudaStream_t st) {
    if (seqs == 0 || max_ctx == 0) return cudaSuccess;
    k_paged_gather<<<dim3((unsigned)max_ctx, (unsigned)seqs), 128, 0, st>>>(kv_heads, hs, block_size, max_blocks, (const uint4 *)pool,
                                                                            tables, lens, seq_offsets, (uint4 *)out);
    return cudaGetLastError();
}

// Copies whole pages inside a K pool and a V pool: pair i copies block map[2i] to block map[2i+1] in both (what a forked
// sequence needs for the one partly filled page it may not share). One CTA per pair, 16-byte accesses.
__global__ void __launch_bounds__(256) k_copy_blocks(uint4 *kpool, uint4 *vpool, const int64_t *__restrict__ map, int64_t vec_per_block) {
    const int64_t src = map[2 * blockIdx.x] * vec_per_block, dst = map[2 * blockIdx.x + 1] * vec_per_block;
    for (int64_t i = threadIdx.x; i < vec_per_block; i += blockDim.x) {
        kpool[dst + i] = kpool[src + i];
        vpool[dst + i] = vpool[src + i];
    }
}
cudaError_t launch_copy_blocks(void *kpool, void *vpool, const int64_t *map_dev, int n_pairs, int64_t bytes_per_block, cudaStream_t st) {
    if (n_pairs == 0) return cudaSuccess;
    k_copy_blocks<<<n_pairs, 256, 0, st>>>((uint4 *)kpool, (uint4 *)vpool, map_dev, bytes_per_block / 16);
    return cudaGetLastError();
}

}  // namespace tlb

// ---------------------------------------------------------------- paged attention without any allocation
// Some callers may not allocate device memory at all: a serving loop that must never touch the
// allocator on its latency path, a host that runs under a fixed memory reservation it does not
// control, code running while another library owns the allocator. For them the split-context
// partial sums (the only scratch paged attention needs) live in this fixed array. It is part of
// the library image: every GPU that loads the library holds these bytes until the process exits.
#define TLB_PA_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_pa_static_scratch[TLB_PA_STATIC_SCRATCH_BYTES];
static __device__ int g_pa_static_err;   // error word of the launches of tlb_paged_attention_static (zero at load)

namespace tlb {
// In host code the array's name is only a handle for the runtime, not a device address; the address
// is looked up once per device, with that device current, and cached here.
static void *g_pa_scratch_addr[64] = {nullptr};
static cudaError_t pa_static_scratch(int ordinal, void **out) {
    if (ordinal < 0 || ordinal >= 64) return cudaErrorInvalidDevice;
    if (!g_pa_scratch_addr[ordinal]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_pa_static_scratch);
        if (e != cudaSuccess) return e;
        g_pa_scratch_addr[ordinal] = p;
    }
    *out = g_pa_scratch_addr[ordinal];
    return cudaSuccess;
}
}  // namespace tlb

extern "C" tlb_status tlb_paged_attention_static(tlb_device *dev, const void *q, const void *k_pool, const void *v_pool,
                                                 const int32_t *block_tables, const int32_t *context_lens, void *out, int seqs,
                                                 int heads, int kv_heads, int head_size, int block_size, int max_blocks,
                                                 int max_context, float scale) {
    using namespace tlb;
    if (!dev || !q || !k_pool || !v_pool || !block_tables || !context_lens || !out)
        return fail(TLB_INVALID, "tlb_paged_attention_static: null argument");
    PagedGeom g{};
    g.seqs = seqs;
    g.heads = heads;
    g.kv_heads = kv_heads;
    g.hs = head_size;
    g.block_size = block_size;
    g.max_ctx = max_context;
    g.max_blocks = max_blocks;
    g.scale = scale;
    if (seqs < 0 || heads < 1 || max_context < 1 || !paged_supported(g))
        return fail(TLB_UNSUPPORTED, "tlb_paged_attention_static: head size must be 64, 128 or 256, the block size a power of two and the query heads a multiple of the kv heads");
    if ((int64_t)max_blocks * block_size < max_context) return fail(TLB_INVALID, "block tables are shorter than the maximum context");
    if (cudaSetDevice(dev->ordinal) != cudaSuccess) return fail(TLB_NO_DEVICE, "cannot make the device current");
    paged_plan(g, dev->prop.multiProcessorCount);
    const uint64_t need = paged_scratch_bytes(g);
    if (need > TLB_PA_STATIC_SCRATCH_BYTES)
        return fail(TLB_INVALID, "tlb_paged_attention_static: this shape needs " + std::to_string(need) + " bytes of scratch, the built-in scratch holds " +
                                     std::to_string((uint64_t)TLB_PA_STATIC_SCRATCH_BYTES) + "; use a compiled program (tlb_program_run) for it");
    void *scratch = nullptr;
    cudaError_t e = pa_static_scratch(dev->ordinal, &scratch);
    if (e != cudaSuccess) return fail(TLB_EXECUTION, "cudaGetSymbolAddress: " + cuda_msg(e));
    int *errw = nullptr;
    e = cudaGetSymbolAddress((void **)&errw, g_pa_static_err);
    if (e != cudaSuccess) return fail(TLB_EXECUTION, "cudaGetSymbolAddress: " + cuda_msg(e));
    // nothing in the scratch has to start at zero: every chunk that the reduce reads is written by this launch.
    // The pools' size is not an argument of this call: lengths are cut to the table row, block ids checked for sign.
    e = launch_paged_attention(g, q, k_pool, v_pool, block_tables, context_lens, out, scratch, 0, errw, dev->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    int flag = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&flag, errw, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, "tlb_paged_attention_static: " + cuda_msg(e));
    }
    if (flag != 0) {
        cudaMemset(errw, 0, 4);
        return fail(TLB_EXECUTION, "tlb_paged_attention_static: a context length or block id from the caller was out of range (skipped on the device)");
    }
    return TLB_OK;
}
