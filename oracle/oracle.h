/* TEST INFRASTRUCTURE ONLY -- the product library never includes, links or calls this.
 *
 * Plain-C restatement of the algorithms on tensorlisp's Device::Native hot path, as the
 * reference's vendored ggml CPU code defines them. Parity is PINNED: tests/test_oracle_vs_ref.py
 * checks every function here against the reference's own ggml build (oracle/_ref, built from the
 * reference checkout by oracle/build.py) and against the fixtures under tests/golden/ that were
 * generated from that build (tests/golden/make_golden.py).
 *
 * Citations are paths inside the reference project. */
#ifndef TLB_ORACLE_H
#define TLB_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q4_1 = 3, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8, ORC_Q2_K = 10, ORC_Q3_K = 11, ORC_Q4_K = 12,
       ORC_Q5_K = 13, ORC_Q6_K = 14, ORC_BF16 = 30 };

uint16_t orc_f32_to_f16(float f);
float    orc_f16_to_f32(uint16_t h);

/* bytes of one row of ne0 elements (vendor/ggml/src/ggml.c ggml_row_size) */
int64_t orc_row_size(int type, int64_t ne0);

/* row quantizers = `tl quantize` (crates/tensorlisp/src/dtype.rs:98-124 -> ggml_quantize_chunk) */
void orc_quantize_row_q8_0(const float *x, void *y, int64_t k); /* ggml-quants.c:276-299  */
void orc_quantize_row_q4_0(const float *x, void *y, int64_t k); /* ggml-quants.c:113-148  */
void orc_quantize_row_q4_K(const float *x, void *y, int64_t k); /* ggml-quants.c:1457-1527 */
void orc_quantize_row_q8_K(const float *x, void *y, int64_t k); /* ggml-quants.c:2768-2805 */
void orc_quantize_row_q4_1(const float *x, void *y, int64_t k); /* ggml-quants.c:150-185   */
void orc_quantize_row_q5_0(const float *x, void *y, int64_t k); /* ggml-quants.c:187-229   */
void orc_quantize_row_q5_1(const float *x, void *y, int64_t k); /* ggml-quants.c:231-273   */
void orc_quantize_row_q2_K(const float *x, void *y, int64_t k); /* ggml-quants.c:891-958   */
void orc_quantize_row_q3_K(const float *x, void *y, int64_t k); /* ggml-quants.c:1229-1303 */
void orc_quantize_row_q5_K(const float *x, void *y, int64_t k); /* ggml-quants.c:1644-1727 */
void orc_quantize_row_q6_K(const float *x, void *y, int64_t k); /* ggml-quants.c:1869-1937 */
int  orc_quantize_rows(int type, const float *src, int64_t nrows, int64_t n_per_row, void *dst);
int  orc_dequantize_row(int type, const void *src, float *dst, int64_t k);

/* y[m + M*n] = vec_dot(W row m, quantized x column n): ggml-cpu's mul_mat with quantized
 * weights (ggml-cpu.c:1272-1357 + generic dots in ggml-cpu/quants.c). x is f32 [K, N]. */
int orc_mul_mat(int type, const void *W, int64_t K, int64_t M, const float *x, int64_t N, float *y);
/* exact dequantized weights times x, accumulated in double (what the reference's own
 * native test compares against, crates/tensorlisp/tests/native.rs:87-102) */
int orc_mul_mat_dequant(int type, const void *W, int64_t K, int64_t M, const float *x, int64_t N, float *y);

/* RMS_NORM (ops.cpp:3794-3860), optionally times a weight row (nn:rms-norm, stdlib/nn.ss:38-43) */
void orc_rms_norm(const float *x, int64_t n, int64_t rows, float eps, const float *w, float *y);
/* SiLU(g)*u (vec.h:1046-1048 + MUL) */
void orc_silu_mul(const float *g, const float *u, int64_t n, float *y);
/* ROPE, modes 0 (normal) and 2 (neox), no YaRN (ext_factor 0), ops.cpp:5822-6093.
 * x is [ne0, heads, tokens]; pos has one entry per token. */
void orc_rope(const float *x, int64_t ne0, int64_t heads, int64_t tokens, const int32_t *pos, int n_dims,
              int mode, float freq_base, float freq_scale, float attn_factor, float *y);
/* SOFT_MAX over rows with a scale, no mask (ops.cpp:5517-5554) */
void orc_soft_max(const float *x, int64_t n, int64_t rows, float scale, float *y);
/* GET_ROWS from a quantized or f32 table */
int orc_get_rows(int type, const void *table, int64_t ne0, const int32_t *ids, int64_t n_ids, float *y);
/* ARGMAX, last index among ties (vec.h ggml_vec_argmax_f32) */
void orc_argmax(const float *x, int64_t n, int64_t rows, int32_t *out);

/* Decode attention of one query token per sequence over dense f16 K/V with an f32 accumulator:
 * out[s,h,:] = softmax(scale * q[s,h,:] . K[s, kvh(h), t, :]) V  (the closed form the reference's
 * paged-attention test uses, crates/kernels/tests/paged_attn_cuda.rs:204-232).
 * q, out: f16 [seqs, heads, hs]; K, V for sequence s start at k[s]/v[s]: f16 [ctx[s], kv_heads, hs]. */
void orc_attention_decode(const uint16_t *q, const uint16_t *const *k, const uint16_t *const *v,
                          const int32_t *ctx, int seqs, int heads, int kv_heads, int hs, float scale,
                          uint16_t *out, float *out_f32);

#ifdef __cplusplus
}
#endif
#endif
