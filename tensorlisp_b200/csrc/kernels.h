// Launch helpers exported by the kernel files (k_*.cu) to the lowering code.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/tlb200.h"

namespace tlb {

// A strided view of up to four dimensions, in bytes, as ggml describes tensors.
struct TView {
    int64_t ne[4];
    int64_t nb[4];
};

// ---------------------------------------------------------------- k_quant.cu
enum { ACT_Q8_0 = 0, ACT_Q8_K = 1 };
struct ActLayout {
    int kind;
    int64_t K, N;
    uint64_t qs_off, d_off, bsum_off, bytes;
};
ActLayout act_layout(int kind, int64_t K, int64_t N);
cudaError_t launch_quantize_rows(uint32_t type, const float *x, int64_t rows, int64_t n_per_row, void *y, cudaStream_t st);
cudaError_t launch_act_quantize(const ActLayout &a, const float *x, int64_t ldx, void *out, cudaStream_t st);

// ---------------------------------------------------------------- k_mm.cu
// y[n*ldy + m] = dot(W row m, quantized activation column n), contiguous W rows of K elements.
// Returns cudaErrorNotSupported when the shape cannot use the pipelined kernel (caller falls back).
bool gemv_supported(uint32_t type, int64_t K, int64_t M, int64_t N);
cudaError_t launch_gemv(uint32_t type, const void *W, int64_t K, int64_t M, const ActLayout &a, const void *act,
                        float *y, int64_t ldy, int sm_count, int *err_flag, cudaStream_t st);
// Generic strided / batched product (any supported weight type, f32 activations or a quantized
// activation block per (i2,i3) batch). dst f32.
struct MMGeneric {
    uint32_t wtype;
    TView w, x, y;       // x: f32 activations (used for plain weight types)
    int64_t r2, r3;      // broadcast ratios
    const void *act;     // quantized activations of the whole x (N = ne1*ne2*ne3 columns), or null
    ActLayout a;
};
cudaError_t launch_mm_generic(const MMGeneric &p, const void *W, const void *X, void *Y, cudaStream_t st);
void gemv_configure();  // sets the dynamic shared-memory attributes once per process

// ---------------------------------------------------------------- k_mmq_tc.cu
// Q4_K weights x 5..64 activation columns on tcgen05 (f16 operands built from the integer codes).
struct TcPlan {
    int npad, nsb, n_split, sb_per_split;
    int streamk;             // > 0: that many CTAs share all (row tile, super-block) units equally (k_mmq_tc.cu)
    int n_col_chunks;        // activation columns are processed npad at a time: one launch per chunk
    uint64_t blob_unit;      // bytes of one packed blob (one chunk of columns, one super-block / stage)
    uint64_t blob_bytes;     // packed activation blobs: [chunk][super-block] x blob_unit
    uint64_t partial_bytes;  // scratch for the K-split partial sums (0 when not split)
};
bool mmq_tc_supported(uint32_t type, int64_t K, int64_t M, int64_t N);
TcPlan mmq_tc_plan(int64_t K, int64_t M, int64_t N, int sm_count);
cudaError_t launch_act_pack_tc(const ActLayout &a, const void *act, int npad, void *blobs, cudaStream_t st);
// leave_partial: with a K split, do not add the partial sums [split][N][M] up (the caller's next kernel does)
cudaError_t launch_mmq_tc(const TcPlan &t, const void *W, int64_t K, int64_t M, int64_t N, const void *blobs, float *y,
                          int64_t ldy, void *partial, int *err, cudaStream_t st, bool leave_partial = false);
// up to 3 matrices [M[j] x K] that share the activations in one launch; outputs dense [N][M[j]]
cudaError_t launch_mmq_tc_group(const TcPlan &t, int n_mats, const void *const *W, int64_t K, const int64_t *M, int64_t N, const void *blobs,
                                float *const *y, int64_t ldy, void *partial, int *err, cudaStream_t st, bool leave_partial = false);
void mmq_tc_configure();
bool tc_available();
cudaError_t launch_wait_runs_out(uint32_t limit, unsigned nap_ns, int *err, unsigned long long *ns, cudaStream_t st);   // the driver offers cuTensorMapEncodeTiled

// ---------------------------------------------------------------- k_mmq_tc_q8.cu
// Q8_0 weights x 5..32 activation columns on tcgen05 (kind::i8, one accumulator per 32-element block).
bool mmq_tc8_supported(int64_t K, int64_t M, int64_t N);
TcPlan mmq_tc8_plan(int64_t K, int64_t M, int64_t N, int sm_count);
cudaError_t launch_act_pack_tc8(const ActLayout &a, const void *act, int npad, void *blobs, cudaStream_t st);
cudaError_t launch_mmq_tc8(const TcPlan &t, const void *W, int64_t K, int64_t M, int64_t N, const void *blobs, float *y,
                           int64_t ldy, void *partial, int *err, cudaStream_t st);
void mmq_tc8_configure();
// the folded-scale prompt GEMM (k_mm_q80_f16) for Q8_0 or Q4_K weights: blobs of 256 columns x 64 elements, f16(code x scale)
constexpr int MM_FOLD_NPAD = 256;
uint64_t mm_fold_blob_unit();   // bytes of the blobs of one 256-element unit of K (four stages)
cudaError_t launch_mm_fold_f16(bool q4k, const void *W, int64_t K, int64_t M, int64_t N, const void *blobs, float *y, int64_t ldy, int *err,
                               cudaStream_t st);
cudaError_t launch_act_pack_fold(const ActLayout &a, const void *act, void *blobs, cudaStream_t st);

// ---------------------------------------------------------------- k_fused.cu
// One row (= activation column n) per CTA: produce the f32 row, quantize it to Q8_K into an ActLayout
// block at `out`, optionally also pack the tensor-core blobs behind it.
enum { RQ_PLAIN = 0, RQ_NORM = 1, RQ_GLU = 2, RQ_F16 = 3 };
struct RowQuantArgs {
    int mode;
    int64_t K, N;
    const float *a;      // PLAIN/NORM: the row source; GLU: gate; F16: half values (cast pointer)
    int64_t lda;
    const float *b;      // PLAIN/NORM: optional addend (residual add), GLU: up
    int64_t ldb;
    float *sum_out;      // a + b written back (new residual stream), may be null
    int64_t ld_sum;
    const float *w;      // NORM: weight row of wn values
    int64_t wn;
    float eps;
    float *y_out;        // optional f32 copy of the produced row
    int64_t ld_y;
    void *out;           // ActLayout block (ACT_Q8_K) for N columns
    uint64_t qs_off, d_off, bsum_off;
    int npad;            // > 0: also pack blobs of npad columns at out + blob_off
    uint64_t blob_off, blob_bytes;
    int q80;             // 0: Q8_K (the default). 1: Q8_0 for the prompt mul_mat of Q8_0 weights: only its packed f16
                         // operand (blobs of 256 columns x 64 elements, value = code x f16 scale) is produced
};
bool row_quant_supported(int64_t K);
bool row_quant_q80_supported(int64_t K, int mode);
cudaError_t launch_row_quant(const RowQuantArgs &p, cudaStream_t st);
// the all-reduce in front of a residual add + RMS norm + quantizer fused into one kernel (tensor parallelism):
// p as for launch_row_quant in RQ_NORM mode with p.a the residual stream; the addend is the all-reduced `a`
struct ArRank;
bool exchange_row_quant_supported(int64_t K, int64_t N);
cudaError_t launch_exchange_row_quant(const ArRank &a, const RowQuantArgs &p, int n_ranks, cudaStream_t st);
cudaError_t launch_exchange_row_quant_emulated(const ArRank *a, const RowQuantArgs *p, int n_ranks, cudaStream_t st);

// ---------------------------------------------------------------- k_core.cu
struct BinArgs { TView a, b, d; int op; };  // 0 add 1 sub 2 mul 3 div; all f32
cudaError_t launch_bin(const BinArgs &p, const void *a, const void *b, void *d, cudaStream_t st);
struct UnaryArgs { TView a, d; int code; float p0, p1; uint32_t aty, dty; };
cudaError_t launch_unary(const UnaryArgs &p, const void *a, void *d, cudaStream_t st);
// GLU: d = act(a) * b over contiguous rows; glu_op as ggml (0 reglu, 1 geglu, 2 swiglu, 4 geglu_erf, 5 geglu_quick)
struct GluArgs { int64_t n, rows; int64_t lda, ldb; int glu_op; };
cudaError_t launch_glu(const GluArgs &p, const float *a, const float *b, float *d, cudaStream_t st);
// (RMS_)NORM over rows of n f32 values, optional multiply by a broadcast weight row of wn values.
struct NormArgs { TView a, d; int rms; float eps; int has_w; TView w; };
cudaError_t launch_norm(const NormArgs &p, const void *a, const void *w, void *d, cudaStream_t st);
struct RopeArgs {
    TView a, d;
    uint32_t aty, dty;
    int n_dims, mode;
    float freq_scale, ext_factor, attn_factor, theta_scale, corr0, corr1;
    int has_ff;
};
cudaError_t launch_rope(const RopeArgs &p, const void *a, const int32_t *pos, const float *ff, void *d, cudaStream_t st);
// rope(q) -> f16, rope(k) -> key pool, v -> value pool in one launch (k and v as [hs, kv_heads, tokens] f32 views)
struct RopeKvArgs {
    RopeArgs rope;   // a = the f32 query view [hs, heads, tokens]
    TView k, v;
    int heads, kv_heads, hs, block_size, tokens;
    int64_t pool_slots;   // block_size * pages of each pool: a slot at or beyond it is skipped and reported
};
cudaError_t launch_rope_kv(const RopeKvArgs &p, const void *q, const void *k, const void *v, const int32_t *pos, const float *ff,
                           void *q16, void *kpool, void *vpool, const int64_t *slots, int *err, cudaStream_t st);
struct SoftmaxArgs { TView a, m, d; float scale, max_bias, m0, m1; int n_head_log2; int has_mask; uint32_t mty; };
cudaError_t launch_soft_max(const SoftmaxArgs &p, const void *a, const void *m, void *d, cudaStream_t st);
struct RowsArgs { TView a, ids, d; uint32_t aty, idty, dty; };
cudaError_t launch_get_rows(const RowsArgs &p, const void *a, const void *ids, void *d, cudaStream_t st);
cudaError_t launch_set_rows(const RowsArgs &p, const void *rows, const void *ids, void *d, cudaStream_t st);
struct CpyArgs { TView a, d; uint32_t aty, dty; };
cudaError_t launch_cpy(const CpyArgs &p, const void *a, void *d, cudaStream_t st);
cudaError_t launch_argmax(const TView &a, const void *x, int32_t *out, cudaStream_t st);
struct SimpleArgs { TView a, b, d; int64_t i0; float f0, f1; };
cudaError_t launch_concat(const SimpleArgs &p, const void *a, const void *b, void *d, cudaStream_t st);
cudaError_t launch_repeat(const SimpleArgs &p, const void *a, void *d, cudaStream_t st);
cudaError_t launch_sum_rows(const SimpleArgs &p, const void *a, void *d, cudaStream_t st);  // i0: 1 = mean
cudaError_t launch_arange(const SimpleArgs &p, void *d, cudaStream_t st);

// image ops (IM2COL, UPSCALE, POOL_2D, CONV_2D_DW, PAD, PAD_REFLECT_1D): one thread per destination element
struct Im2colArgs { TView x, d; uint32_t xty, dty; int s0, s1, p0, p1, d0, d1, is2d; int64_t KW, KH, IH, IW; };
cudaError_t launch_im2col(const Im2colArgs &p, const void *x, void *d, cudaStream_t st);
struct UpscaleArgs { TView a, d; float sf0, sf1, sf2, sf3, poff; int mode, antialias; };   // f32 -> f32
cudaError_t launch_upscale(const UpscaleArgs &p, const void *a, void *d, cudaStream_t st);
struct Pool2dArgs { TView a, d; uint32_t aty, dty; int kind, k0, k1, s0, s1, p0, p1; };
cudaError_t launch_pool_2d(const Pool2dArgs &p, const void *a, void *d, cudaStream_t st);
struct ConvDwArgs { TView k, x, d; uint32_t kty, xty, dty; int s0, s1, p0, p1, d0, d1; };
cudaError_t launch_conv_2d_dw(const ConvDwArgs &p, const void *k, const void *x, void *d, cudaStream_t st);
struct PadArgs { TView a, d; int64_t lp[4]; int elem_bytes, reflect; };
cudaError_t launch_pad(const PadArgs &p, const void *a, void *d, cudaStream_t st);

// ---------------------------------------------------------------- k_flash.cu
// FLASH_ATTN_EXT (dense): q f32 [d, nq, nh, nb], k / v f16 or f32 [d, nkv, nhkv, nb], optional f16 mask
struct FlashArgs {
    TView q, k, v, m;
    int nq, nkv, nh, nhkv, nb, d, dv, m_ne2, m_ne3, n_head_log2;   // d: head size of queries and keys, dv: of values
    float scale, softcap, max_bias, m0, m1;   // scale already divided by softcap when that is set
    bool k_f32, v_f32;
    uint32_t k_ty, v_ty;   // ggml types of keys and values: f16 / f32 everywhere, bf16 and the block types on the one-query-per-CTA kernel
    // split-KV (few queries over a long cache): the keys are cut into `parts` stretches of part_len, every stretch is a
    // CTA of its own that leaves (maximum, sum, unnormalised output) in scratch, and a second launch merges them
    int part_len, parts;
};
bool flash_supported(int64_t d, int64_t dv);
// 64 / 128 run on the tensor cores from 16-byte copies: their rows must start on 16-byte boundaries
bool flash_rows_need_alignment(int64_t d, int64_t dv);
// fills p.part_len / p.parts (parts = 1: no split) for a device of sm_count SMs; bytes of scratch the split needs
void flash_split_plan(FlashArgs &p, int sm_count);
uint64_t flash_split_scratch_bytes(const FlashArgs &p);
cudaError_t launch_flash_attn(const FlashArgs &p, const void *q, const void *k, const void *v, const void *mask, float *out, void *scratch,
                              cudaStream_t st);
// ---------------------------------------------------------------- k_flash_tc.cu
// The same op on tcgen05 for prompt-sized query counts (head size 128, f16 keys / values, no soft cap, no ALiBi);
// scratch holds the packed operands and the per-tile mask flags.
bool flash_tc_supported(const FlashArgs &p, bool has_mask);
uint64_t flash_tc_scratch_bytes(const FlashArgs &p, bool has_mask);
cudaError_t launch_flash_attn_tc(const FlashArgs &p, const void *q, const void *k, const void *v, const void *mask, float *out, void *scratch,
                                 int *err, cudaStream_t st);
void flash_tc_configure();

// Values of the device error word behind a program's arena: 1-3 are bounded waits that gave up (GEMV copies, tensor-core
// pipelines, the peer exchange); 4 is a context length, block id or cache slot from the caller that a kernel skipped
// because it pointed outside the tables or pools.
#define TLB_ERR_INDEX 4

// ---------------------------------------------------------------- k_attn.cu
// KV pools are private to the executor (only the two paged nodes touch them): f16
// [block][kv_head][slot][head_size] for both keys and values.
struct PagedGeom {
    int seqs, heads, kv_heads, hs, block_size, max_ctx, max_blocks;
    float scale;
    int chunk_tokens, n_chunks;  // split of the context (filled by paged_plan)
};
void paged_plan(PagedGeom &g, int sm_count);
uint64_t paged_scratch_bytes(const PagedGeom &g);
bool paged_supported(const PagedGeom &g);
// rq: also quantize the output rows to Q8_K (RQ_F16 semantics of the row quantizer; needs n_chunks == 1 and
// paged_quant_fusable(g)); null: only the f16 output
struct RowQuantArgs;
bool paged_quant_fusable(const PagedGeom &g);
cudaError_t launch_paged_attention(const PagedGeom &g, const void *q, const void *kpool, const void *vpool,
                                   const int32_t *tables, const int32_t *lens, void *out, void *scratch,
                                   int64_t pool_blocks, int *err, cudaStream_t st, const RowQuantArgs *rq = nullptr);
// pool_slots: block_size * pages of each pool; a slot at or beyond it is skipped and reported through err
cudaError_t launch_cache_write(int tokens, int kv_heads, int hs, int block_size, const void *key, const void *value,
                               void *kpool, void *vpool, const int64_t *slots, int64_t pool_slots, int *err, cudaStream_t st);
// paged pool -> dense f16 [ctx, kv_heads, hs] per sequence, concatenated in sequence order
cudaError_t launch_copy_blocks(void *kpool, void *vpool, const int64_t *map_dev, int n_pairs, int64_t bytes_per_block, cudaStream_t st);
cudaError_t launch_paged_gather(int seqs, int kv_heads, int hs, int block_size, int max_blocks, const void *pool,
                                const int32_t *tables, const int32_t *lens, const int64_t *seq_offsets, void *out,
                                int max_ctx, cudaStream_t st);
void attn_configure();

}  // namespace tlb
