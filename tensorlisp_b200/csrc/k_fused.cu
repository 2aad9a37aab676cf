// Row producers fused with the Q8_K activation quantizer of the next MUL_MAT (and with the packing of
// the tensor-core operand): one launch replaces ADD, RMS_NORM*w (or act(gate)*up, or an f16->f32 cast),
// QUANT_ACT and the blob packer. The reference's CUDA executor fuses nothing (lower.rs:1-6); its
// Tree/Vulkan executors form the same chains on the IR (vulkan/fuse.rs:56-152, fuse_tree.rs: FUSED_ROW,
// FUSED_GU, int8 producer outputs), and list "quantize each distinct activation once by its producer"
// as the next step (docs/design/tree.md:361-364).
//
// Arithmetic is unchanged: the f32 row is produced with the same operations as the separate kernels
// (k_core.cu), then quantized exactly like quantize_row_q8_K_ref (ggml-quants.c:2768-2805). This file
// is compiled with -fmad=false because of the quantizer's rounding.
#include <cuda_fp16.h>

#include "kernels.h"
#include "exchange.cuh"
#include "rowquant.cuh"
#include "pdl.cuh"

namespace tlb {

constexpr int RQ_THREADS = 256;
constexpr int RQ_WARPS = RQ_THREADS / 32;

// The f32 value at (column n, element k) before any normalisation: a, a + b, act(a) * b or f16 a.
__device__ __forceinline__ void rq_load8(const RowQuantArgs &p, int n, int64_t k0, float (&x)[8]) {
    if (p.mode == RQ_GLU) {
        const float4 g0 = *reinterpret_cast<const float4 *>(p.a + n * p.lda + k0), g1 = *reinterpret_cast<const float4 *>(p.a + n * p.lda + k0 + 4);
        const float4 u0 = *reinterpret_cast<const float4 *>(p.b + n * p.ldb + k0), u1 = *reinterpret_cast<const float4 *>(p.b + n * p.ldb + k0 + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int e = 0; e < 8; e++) x[e] = __fmul_rn(__fdiv_rn(g[e], __fadd_rn(1.0f, expf(-g[e]))), u[e]);   // SiLU(g)*u
    } else if (p.mode == RQ_F16) {
        const uint4 h = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(p.a) + n * p.lda + k0);
        const __half2 *h2 = reinterpret_cast<const __half2 *>(&h);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float2 f = __half22float2(h2[e]);
            x[2 * e] = f.x;
            x[2 * e + 1] = f.y;
        }
    } else {
        const float4 a0 = *reinterpret_cast<const float4 *>(p.a + n * p.lda + k0), a1 = *reinterpret_cast<const float4 *>(p.a + n * p.lda + k0 + 4);
        x[0] = a0.x; x[1] = a0.y; x[2] = a0.z; x[3] = a0.w; x[4] = a1.x; x[5] = a1.y; x[6] = a1.z; x[7] = a1.w;
        if (p.b) {   // residual add: x = a + b
            const float4 b0 = *reinterpret_cast<const float4 *>(p.b + n * p.ldb + k0), b1 = *reinterpret_cast<const float4 *>(p.b + n * p.ldb + k0 + 4);
            x[0] = __fadd_rn(x[0], b0.x); x[1] = __fadd_rn(x[1], b0.y); x[2] = __fadd_rn(x[2], b0.z); x[3] = __fadd_rn(x[3], b0.w);
            x[4] = __fadd_rn(x[4], b1.x); x[5] = __fadd_rn(x[5], b1.y); x[6] = __fadd_rn(x[6], b1.z); x[7] = __fadd_rn(x[7], b1.w);
        }
    }
}

// Grid (column, slice of 8 blocks): every warp owns ONE 256-element block, so a row of 4096 (14336)
// elements is spread over 2 (7) CTAs instead of one warp walking several blocks in turn. With a
// normalisation, every CTA of a row first adds up the squares of the whole row in the same order
// (the row is a few KB and sits in L2), so all of them use the same scale.
__global__ void __launch_bounds__(RQ_THREADS) k_row_quant_q8k(RowQuantArgs p) {
    __shared__ float red[RQ_WARPS];
    griddep_launch();
    griddep_wait();
    const int n = blockIdx.x;          // activation column (= token)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t K = p.K;
    const int nblk = (int)(K / 256);
    const int sb = blockIdx.y * RQ_WARPS + warp;
    char *ob = (char *)p.out;
    if (n >= p.N) {
        // padding columns of the tensor-core blobs are zero
        if (p.npad == MM_FOLD_NPAD) {
            if (sb < nblk) {
                const int64_t kk = (int64_t)sb * 256 + lane * 8;
                *reinterpret_cast<uint4 *>((uint8_t *)ob + p.blob_off + ((size_t)(n >> 8) * (size_t)(K / 64) + (size_t)(kk >> 6)) * 32768 +
                                           (size_t)((n & 255) >> 3) * 1024 + (size_t)((kk & 63) >> 3) * 128 + (size_t)(n & 7) * 16) = make_uint4(0, 0, 0, 0);
            }
        } else if (p.npad > 0 && sb < nblk) {
            const int ch = n / p.npad, nl = n % p.npad;   // blobs: [chunk of npad columns][block]
            uint8_t *o = (uint8_t *)ob + p.blob_off + ((size_t)ch * nblk + sb) * p.blob_bytes;
            *reinterpret_cast<uint4 *>(o + (size_t)(nl / 8) * 4096 + lane * 128 + (nl % 8) * 16) = make_uint4(0, 0, 0, 0);
            if ((lane & 1) == 0)
                *reinterpret_cast<__half *>(o + (size_t)p.npad * 512 + (size_t)(nl / 8) * 256 + (lane >> 4) * 128 + (nl % 8) * 16 + ((lane >> 1) & 7) * 2) = __float2half_rn(0.f);
            if (lane == 0) reinterpret_cast<float *>(o + (size_t)p.npad * 544)[nl] = 0.f;
        }
        return;
    }
    float scale = 1.f;
    float v[8];
    bool have = false;   // v already holds this warp's block (met while the whole row was read for the norm)
    if (p.mode == RQ_NORM) {
        // thread t reads elements t*8.. of every 2048-element stretch in turn: in stretch blockIdx.y those are the very
        // values of the block this warp quantizes below, so they are kept instead of being read a second time
        float ss = 0.f;
        int it = 0;
        for (int64_t k0 = (int64_t)threadIdx.x * 8; k0 < K; k0 += RQ_THREADS * 8, it++) {
            float x[8];
            rq_load8(p, n, k0, x);
#pragma unroll
            for (int e = 0; e < 8; e++) ss = __fadd_rn(ss, __fmul_rn(x[e], x[e]));
            if (it == (int)blockIdx.y) {
                have = true;
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = x[e];
            }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < RQ_WARPS; i++) tot = __fadd_rn(tot, red[i]);
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.eps)));
    }
    if (sb >= nblk) return;
    // ---- this warp's block: lane holds 8 consecutive values
    const int64_t k0 = (int64_t)sb * 256 + lane * 8;
    if (!have) rq_load8(p, n, k0, v);
    if (p.mode != RQ_GLU && p.mode != RQ_F16 && p.b && p.sum_out) {   // the sum is the new residual stream
        *reinterpret_cast<float4 *>(p.sum_out + n * p.ld_sum + k0) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p.sum_out + n * p.ld_sum + k0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (p.mode == RQ_NORM) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int wi = p.wn == K ? (int)(k0 + e) : (int)((uint32_t)(k0 + e) % (uint32_t)p.wn);
            v[e] = __fmul_rn(__fmul_rn(v[e], scale), p.w[wi]);
        }
    }
    rq_quant_block(p, n, sb, nblk, lane, v);
}

// ---------------------------------------------------------------- the same producers in front of a Q8_0 quantizer (prompt pass)
// Q8_0 weights against prompt-sized batches read one operand only: f16(code x f16 scale) of the activations' Q8_0
// quantization, packed in blobs of 256 columns x 64 elements of K (k_mm_q80_f16, k_mmq_tc_q8.cu). This kernel
// produces that (and the Q8_0 block itself) from the f32 row source (a, a + b with the sum written back, RMS norm of either, SiLU(g) * u,
// f16 values), so the normalised / gated f32 row never goes to memory. Quantization follows quantize_row_q8_0_ref
// (ggml-quants.c): d = amax / 127 over 32 values, codes roundf(x / d), the scale rounded to f16.
// A lane holds 8 consecutive values (a block is 4 lanes), a warp 256. With a norm ONE CTA owns the row (rows up to 8192
// elements: 32 warps) and the row is read once; without, a row is spread over CTAs of 8 warps.
__global__ void __launch_bounds__(1024) k_row_quant_q80(RowQuantArgs p) {
    __shared__ float red[32];
    griddep_launch();
    griddep_wait();
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int64_t K = p.K;
    const int nblk = (int)(K / 256);
    const int sb = blockIdx.y * nwarps + warp;
    const bool live = sb < nblk;
    const int64_t k0 = (int64_t)sb * 256 + lane * 8;
    // this lane's 16 bytes of the operand: column n of tile n / 256, stage k0 / 64, chunk (k0 % 64) / 8
    uint8_t *blob = (uint8_t *)p.out + p.blob_off + ((size_t)(n >> 8) * (size_t)(K / 64) + (size_t)(k0 >> 6)) * 32768 +
                    (size_t)((n & 255) >> 3) * 1024 + (size_t)((k0 & 63) >> 3) * 128 + (size_t)(n & 7) * 16;
    if (n >= p.N) {   // padding columns of the last tile are zero
        if (live) *reinterpret_cast<uint4 *>(blob) = make_uint4(0, 0, 0, 0);
        return;
    }
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) {
        rq_load8(p, n, k0, v);
        if (p.mode != RQ_GLU && p.mode != RQ_F16 && p.b && p.sum_out) {   // the sum is the new residual stream
            *reinterpret_cast<float4 *>(p.sum_out + n * p.ld_sum + k0) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(p.sum_out + n * p.ld_sum + k0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
    if (p.mode == RQ_NORM) {   // gridDim.y == 1: the whole row is in this CTA's registers
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) ss = __fadd_rn(ss, __fmul_rn(v[e], v[e]));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int i = 0; i < nwarps; i++) tot = __fadd_rn(tot, red[i]);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.eps)));
        if (live) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int wi = p.wn == K ? (int)(k0 + e) : (int)((uint32_t)(k0 + e) % (uint32_t)p.wn);
                v[e] = __fmul_rn(__fmul_rn(v[e], scale), p.w[wi]);
            }
        }
    }
    if (!live) return;
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.f);
    const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.0f;
    const float dh = __half2float(__float2half_rn(d));   // the block's scale as the dot product reads it
    uint32_t h[4];
    int q[8];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float q0 = roundf(__fmul_rn(v[2 * e], id)), q1 = roundf(__fmul_rn(v[2 * e + 1], id));
        q[2 * e] = (int)q0;
        q[2 * e + 1] = (int)q1;
        const __half2 t = __floats2half2_rn(__fmul_rn(q0, dh), __fmul_rn(q1, dh));
        h[e] = *reinterpret_cast<const uint32_t *>(&t);
    }
    *reinterpret_cast<uint4 *>(blob) = make_uint4(h[0], h[1], h[2], h[3]);
    // the Q8_0 block itself too (int8 codes and f32 scales): a consumer that is not a prompt-sized 2-D mul_mat reads those
    uint2 packed;
    packed.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    packed.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>((int8_t *)p.out + p.qs_off + (size_t)n * K + k0) = packed;
    if ((lane & 3) == 0) reinterpret_cast<float *>((char *)p.out + p.d_off)[(size_t)n * (K / 32) + (k0 >> 5)] = dh;
}

bool row_quant_q80_supported(int64_t K, int mode) { return K % 256 == 0 && K >= 256 && (mode != RQ_NORM || K <= 8192); }

// ---------------------------------------------------------------- exchange + residual add + RMS norm + quantizer
// Tensor parallelism: the all-reduce behind a row-parallel projection, the residual add, the RMS norm and the
// Q8_K quantization of the next mul_mat's input as ONE kernel. A CTA owns one activation row (token): it adds up
// the K-split partial sums of its rank (if any), pushes the row into a slot of every peer's exchange buffer with
// plain stores over NVLink, each value in one 8-byte word with the call's sequence number; every thread then waits
// (bounded) for its own eight values of every rank in the local buffer, adds them in rank order (so all ranks hold
// identical sums), and the CTA has the whole reduced row in the registers of its 16 warps: residual add, sum of
// squares, scale, quantize, pack. Slots alternate by call parity as in the plain all-reduce (comm.cu, exchange.cuh);
// this kernel uses the second buffer set, whose flag area it does not need.
constexpr int XR_THREADS = 512;   // 16 warps, one 256-value block each: rows up to 4096 elements

__device__ __forceinline__ void xr_body(const ArRank &a, const RowQuantArgs &p, int n_ranks, int n, int rows) {
    __shared__ float red[RQ_WARPS];
    __shared__ float xs[XR_THREADS / 32 - RQ_WARPS][32][9];   // values of warps 8..15, handed to warps 0..7 (padded rows)
    __shared__ int s_fail;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t K = p.K;
    const int nblk = (int)(K / 256);
    if (n >= p.N) {   // padding columns of the tensor-core blobs are zero; they take no part in the exchange
        if (p.npad > 0 && warp < nblk) {
            const int ch = n / p.npad, nl = n % p.npad;
            uint8_t *o = (uint8_t *)p.out + p.blob_off + ((size_t)ch * nblk + warp) * p.blob_bytes;
            *reinterpret_cast<uint4 *>(o + (size_t)(nl / 8) * 4096 + lane * 128 + (nl % 8) * 16) = make_uint4(0, 0, 0, 0);
            if ((lane & 1) == 0)
                *reinterpret_cast<__half *>(o + (size_t)p.npad * 512 + (size_t)(nl / 8) * 256 + (lane >> 4) * 128 + (nl % 8) * 16 + ((lane >> 1) & 7) * 2) = __float2half_rn(0.f);
            if (lane == 0) reinterpret_cast<float *>(o + (size_t)p.npad * 544)[nl] = 0.f;
        }
        return;
    }
    if (a.skip_push) return;   // self tests: a rank that never shows up
    char *local = a.peer[a.rank] + AR_SET_BYTES;   // second set: this kernel cuts the data by rows
    uint32_t *seqs = reinterpret_cast<uint32_t *>(local + AR_SEQ_OFF);
    const uint32_t seq = seqs[n] + 1, par = seq & 1;
    const bool live = warp < nblk;
    const int64_t e0 = (int64_t)n * K + warp * 256 + lane * 8;   // this lane's 8 elements of the [rows][K] matrix
    if (tid == 0) s_fail = 0;
    float b[8];
    if (live) {
        const float *src = (a.n_split > 0 ? a.partial : a.data) + e0;
        float4 b0 = *reinterpret_cast<const float4 *>(src), b1 = *reinterpret_cast<const float4 *>(src + 4);
        for (int s = 1; s < a.n_split; s++) {   // K-split partial sums of this rank, in split order
            const float *ps = src + (size_t)s * rows * K;
            const float4 c0 = *reinterpret_cast<const float4 *>(ps), c1 = *reinterpret_cast<const float4 *>(ps + 4);
            b0.x = __fadd_rn(b0.x, c0.x); b0.y = __fadd_rn(b0.y, c0.y); b0.z = __fadd_rn(b0.z, c0.z); b0.w = __fadd_rn(b0.w, c0.w);
            b1.x = __fadd_rn(b1.x, c1.x); b1.y = __fadd_rn(b1.y, c1.y); b1.z = __fadd_rn(b1.z, c1.z); b1.w = __fadd_rn(b1.w, c1.w);
        }
        if (a.flagged_words) {
            // Every value travels with the call's sequence number in the same 8-byte word (the data slots then hold
            // {f32, u32} pairs), so there is no fence, no separate flag and no second round trip: a reader that sees
            // the number sees the value. An aligned 8-byte store is not torn on the way. Twice the bytes on the wire.
            const size_t off = AR_SET_BYTES + AR_DATA_OFF + ((size_t)par * AR_MAX_RANKS + a.rank) * AR_SLOT_BYTES + (size_t)e0 * 8;
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            for (int r = 0; r < n_ranks; r++) {
                char *dst = a.peer[r] + off;
#pragma unroll
                for (int e = 0; e < 8; e += 2)
                    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + e * 8), "r"(__float_as_uint(bv[e])), "r"(seq),
                                 "r"(__float_as_uint(bv[e + 1])), "r"(seq)
                                 : "memory");
            }
        } else {
            const size_t off = AR_SET_BYTES + AR_DATA_OFF + ((size_t)par * AR_MAX_RANKS + a.rank) * AR_SLOT_BYTES + (size_t)e0 * 4;
            for (int r = 0; r < n_ranks; r++) {
                float4 *dst = reinterpret_cast<float4 *>(a.peer[r] + off);
                dst[0] = b0;
                dst[1] = b1;
            }
        }
    }
    if (!a.flagged_words) __threadfence_system();
    __syncthreads();   // (s_fail is initialised for everybody)
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float ss = 0.f;
    const int64_t k0 = (int64_t)warp * 256 + lane * 8;
    float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (a.flagged_words) {
        // ---- wait (bounded) for this thread's eight values of every rank in the local slots, add them in rank order
        if (live) {
            const char *slots = local + AR_DATA_OFF + (size_t)par * AR_MAX_RANKS * AR_SLOT_BYTES + (size_t)e0 * 8;
            bool gave_up = false;
            for (int r = 0; r < n_ranks && !gave_up; r++) {
                const char *src = slots + (size_t)r * AR_SLOT_BYTES;
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    uint32_t d0 = 0, f0 = 0, d1 = 0, f1 = 0, it = 0;
                    for (;;) {
                        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1) : "l"(src + e * 8) : "memory");
                        if (f0 == seq && f1 == seq) break;
                        if (++it >= a.spin_limit || *(volatile int *)&s_fail) { gave_up = true; break; }
                        __nanosleep(100);   // sixteen thousand threads polling without a pause hold up the writes they wait for
                    }
                    // rank 0's values start the sums (0 + x would turn -0 into +0)
                    s8[e] = r == 0 ? __uint_as_float(d0) : __fadd_rn(s8[e], __uint_as_float(d0));
                    s8[e + 1] = r == 0 ? __uint_as_float(d1) : __fadd_rn(s8[e + 1], __uint_as_float(d1));
                }
            }
            if (gave_up) s_fail = 1;
        }
    } else {
        // ---- one flag per (rank, row): raised behind the fence above, awaited (bounded) by one thread per rank
        if (tid < n_ranks) {
            uint32_t *flag = reinterpret_cast<uint32_t *>(a.peer[tid] + AR_SET_BYTES + AR_FLAG_OFF) + ((size_t)par * AR_MAX_RANKS + a.rank) * AR_CTAS + n;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
            const uint32_t *mine = reinterpret_cast<const uint32_t *>(local + AR_FLAG_OFF) + ((size_t)par * AR_MAX_RANKS + tid) * AR_CTAS + n;
            bool ok = false;
            for (uint32_t it = 0; it < a.spin_limit; it++) {
                uint32_t f;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(mine) : "memory");
                if ((int32_t)(f - seq) >= 0) { ok = true; break; }
            }
            if (!ok) s_fail = 1;
        }
        __syncthreads();
        // the slots in rank order (L2 loads: L1 may hold this slot's lines of two calls ago)
        if (live && !s_fail) {
            const char *slots = local + AR_DATA_OFF + (size_t)par * AR_MAX_RANKS * AR_SLOT_BYTES + (size_t)e0 * 4;
            for (int r = 0; r < n_ranks; r++) {
                const float4 c0 = __ldcg(reinterpret_cast<const float4 *>(slots + (size_t)r * AR_SLOT_BYTES));
                const float4 c1 = __ldcg(reinterpret_cast<const float4 *>(slots + (size_t)r * AR_SLOT_BYTES) + 1);
                const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                for (int e = 0; e < 8; e++) s8[e] = r == 0 ? cv[e] : __fadd_rn(s8[e], cv[e]);
            }
        }
    }
    __syncthreads();
    if (s_fail) {
        if (tid == 0) {
            atomicExch(a.err, 3);
            seqs[n] = seq;
        }
        return;
    }
    if (live) {
        const float4 s0 = make_float4(s8[0], s8[1], s8[2], s8[3]), s1 = make_float4(s8[4], s8[5], s8[6], s8[7]);
        const float4 a0 = *reinterpret_cast<const float4 *>(p.a + n * p.lda + k0), a1 = *reinterpret_cast<const float4 *>(p.a + n * p.lda + k0 + 4);
        v[0] = __fadd_rn(a0.x, s0.x); v[1] = __fadd_rn(a0.y, s0.y); v[2] = __fadd_rn(a0.z, s0.z); v[3] = __fadd_rn(a0.w, s0.w);
        v[4] = __fadd_rn(a1.x, s1.x); v[5] = __fadd_rn(a1.y, s1.y); v[6] = __fadd_rn(a1.z, s1.z); v[7] = __fadd_rn(a1.w, s1.w);
        if (p.sum_out) {   // the new residual stream
            *reinterpret_cast<float4 *>(p.sum_out + n * p.ld_sum + k0) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(p.sum_out + n * p.ld_sum + k0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
    // ---- RMS norm over the row. The squares are added in the order of k_row_quant_q8k (256 threads, thread t
    // takes elements t*8.. of every 2048-element stretch in turn, then a shuffle tree, then the 8 warp sums in
    // order), so this kernel and the unfused pair of launches give the same bits: warps 8..15 hand their values
    // to the warps that would have read them in the second pass.
    if (warp >= RQ_WARPS) {
#pragma unroll
        for (int e = 0; e < 8; e++) xs[warp - RQ_WARPS][lane][e] = v[e];
    }
    __syncthreads();
    if (warp < RQ_WARPS) {
#pragma unroll
        for (int e = 0; e < 8; e++) ss = __fadd_rn(ss, __fmul_rn(v[e], v[e]));
        if (warp + RQ_WARPS < nblk) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float x = xs[warp][lane][e];
                ss = __fadd_rn(ss, __fmul_rn(x, x));
            }
        }
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, sft));
        if (lane == 0) red[warp] = ss;
    }
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < RQ_WARPS; i++) tot = __fadd_rn(tot, red[i]);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.eps)));
    if (live) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int wi = p.wn == K ? (int)(k0 + e) : (int)((uint32_t)(k0 + e) % (uint32_t)p.wn);
            v[e] = __fmul_rn(__fmul_rn(v[e], scale), p.w[wi]);
        }
        rq_quant_block(p, n, warp, nblk, lane, v);
    }
    if (tid == 0) seqs[n] = seq;
}

__global__ void __launch_bounds__(XR_THREADS) k_exchange_row_quant(ArRank a, RowQuantArgs p, int n_ranks) {
    // the mul_mat behind this kernel may start and prefetch its weights while the ranks exchange their rows (it waits
    // for this grid before it touches the activations); the trigger fires once every CTA of this grid is running
    griddep_launch();
    griddep_wait();
    xr_body(a, p, n_ranks, blockIdx.x, (int)p.N);
}
// All ranks in ONE cooperative launch on one GPU (blockIdx.y = rank): the single-GPU test of the fused kernel
struct XrAll {
    ArRank a[4];
    RowQuantArgs p[4];
};
__global__ void __launch_bounds__(XR_THREADS) k_exchange_row_quant_emulated(XrAll all, int n_ranks) {
    xr_body(all.a[blockIdx.y], all.p[blockIdx.y], n_ranks, blockIdx.x, (int)all.p[blockIdx.y].N);
}

// (with flagged words a slot holds {value, sequence number} pairs: 8 bytes per element)
bool exchange_row_quant_supported(int64_t K, int64_t N) { return K % 256 == 0 && K / 256 <= XR_THREADS / 32 && N >= 1 && N <= AR_CTAS && N * K * 8 <= (int64_t)AR_SLOT_BYTES; }

static int xr_rows(const RowQuantArgs &p) { return p.npad > 0 ? (int)((p.N + p.npad - 1) / p.npad) * p.npad : (int)p.N; }

cudaError_t launch_exchange_row_quant(const ArRank &a, const RowQuantArgs &p, int n_ranks, cudaStream_t st) {
    return launch_pdl(k_exchange_row_quant, dim3((unsigned)xr_rows(p)), dim3(XR_THREADS), 0, st, a, p, n_ranks);
}

// n_ranks <= 4 emulated ranks, one cooperative launch
cudaError_t launch_exchange_row_quant_emulated(const ArRank *a, const RowQuantArgs *p, int n_ranks, cudaStream_t st) {
    if (n_ranks < 1 || n_ranks > 4) return cudaErrorInvalidValue;
    XrAll all{};
    for (int r = 0; r < n_ranks; r++) {
        all.a[r] = a[r];
        all.p[r] = p[r];
    }
    void *args[] = {&all, &n_ranks};
    return cudaLaunchCooperativeKernel((void *)k_exchange_row_quant_emulated, dim3(xr_rows(p[0]), n_ranks), dim3(XR_THREADS), args, 0, st);
}

bool row_quant_supported(int64_t K) { return K % 256 == 0 && K / 256 <= 65535 * RQ_WARPS; }

cudaError_t launch_row_quant(const RowQuantArgs &p, cudaStream_t st) {
    if (p.N == 0 || p.K == 0) return cudaSuccess;
    if (p.q80) {
        if (p.npad != 256 || !row_quant_q80_supported(p.K, p.mode)) return cudaErrorInvalidValue;
        const int rows256 = (int)((p.N + 255) / 256) * 256, nb = (int)(p.K / 256);
        if (p.mode == RQ_NORM) return launch_pdl(k_row_quant_q80, dim3(rows256, 1), dim3(nb * 32), 0, st, p);
        return launch_pdl(k_row_quant_q80, dim3(rows256, (nb + 7) / 8), dim3(256), 0, st, p);
    }
    const int rows = p.npad > 0 ? (int)((p.N + p.npad - 1) / p.npad) * p.npad : (int)p.N;   // padding columns of the last chunk too
    const int nblk = (int)(p.K / 256);
    return launch_pdl(k_row_quant_q8k, dim3(rows, (nblk + RQ_WARPS - 1) / RQ_WARPS), dim3(RQ_THREADS), 0, st, p);
}

}  // namespace tlb
