// TEST INFRASTRUCTURE ONLY -- never linked into or called from the product library.
//
// A thin C interface over the reference's own vendored ggml (CPU backend + row
// quantizers), compiled by oracle/Makefile from the sources where they lie in the
// reference checkout (vendor/ggml/src, file list of crates/ggml-sys/build.rs:357-418).
// It lets tests and the CPU-baseline leg of bench.py
//   * quantize / dequantize rows with ggml_quantize_chunk and the type traits
//     (what crates/tensorlisp/src/dtype.rs:98-124 calls),
//   * build a ggml graph from a small op list through the public ggml C API (what the
//     generated Scheme ops wrap 1:1, README.md:120-123) and compute it on the CPU
//     backend with a thread count, exactly as Device::Cpu does
//     (crates/tensorlisp/src/model.rs:430-436),
//   * read back every tensor's metadata (type, ne, nb, op name, op_params, sources,
//     view_src/view_offs) the way crates/tensorlisp/src/native_ir.rs:41-95 reads it,
//     so the product's own graph builder can be checked against ggml's shape inference.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "ggml.h"
#include "gguf.h"
#include "ggml-cpu.h"
#include "ggml-backend.h"

extern "C" {
// declared in ggml-cpu/quants.h (not a public header)
void quantize_row_q8_0(const float * x, void * y, int64_t k);
void quantize_row_q8_K(const float * x, void * y, int64_t k);
}

struct tlref_ctx {
    ggml_context * ctx = nullptr;
    std::vector<ggml_tensor *> t;
    int n_threads = 1;
    ggml_backend_t cpu = nullptr;
    std::string err;
};

static int push(tlref_ctx * c, ggml_tensor * x) {
    if (!x) return -1;
    c->t.push_back(x);
    return (int)c->t.size() - 1;
}

extern "C" {

int64_t tlref_row_size(int type, int64_t ne0) { return (int64_t)ggml_row_size((ggml_type)type, ne0); }

// f32 rows -> blocks, as `tl quantize` does it (ggml.c:7952).
int64_t tlref_quantize(int type, const float * src, void * dst, int64_t nrows, int64_t n_per_row) {
    return (int64_t)ggml_quantize_chunk((ggml_type)type, src, dst, 0, nrows, n_per_row, nullptr);
}

int tlref_dequantize(int type, const void * src, float * dst, int64_t n) {
    const ggml_type_traits * tr = ggml_get_type_traits((ggml_type)type);
    if (!tr || !tr->to_float) return -1;
    tr->to_float(src, dst, n);
    return 0;
}

// The activation quantizers ggml-cpu's mul_mat applies to src1 (ggml-cpu.c:1272-1357).
void tlref_act_q8_0(const float * x, void * y, int64_t k) { quantize_row_q8_0(x, y, k); }
void tlref_act_q8_K(const float * x, void * y, int64_t k) { quantize_row_q8_K(x, y, k); }

tlref_ctx * tlref_new(uint64_t mem_bytes, int n_threads) {
    ggml_init_params p = { (size_t)mem_bytes, nullptr, false };
    tlref_ctx * c = new tlref_ctx;
    c->ctx = ggml_init(p);
    c->n_threads = n_threads > 0 ? n_threads : 1;
    if (!c->ctx) { delete c; return nullptr; }
    return c;
}

void tlref_free(tlref_ctx * c) {
    if (!c) return;
    if (c->cpu) ggml_backend_free(c->cpu);
    ggml_free(c->ctx);
    delete c;
}

const char * tlref_error(tlref_ctx * c) { return c->err.c_str(); }

int tlref_tensor(tlref_ctx * c, int type, const int64_t * ne, const char * name) {
    ggml_tensor * x = ggml_new_tensor_4d(c->ctx, (ggml_type)type, ne[0], ne[1], ne[2], ne[3]);
    if (x && name) ggml_set_name(x, name);
    return push(c, x);
}

void * tlref_data(tlref_ctx * c, int id) { return c->t[id]->data; }
uint64_t tlref_nbytes(tlref_ctx * c, int id) { return ggml_nbytes(c->t[id]); }

// op: lower-case ggml constructor name without the ggml_ prefix.
int tlref_op(tlref_ctx * c, const char * op, const int * src, int nsrc, const int64_t * ia, int ni,
             const float * fa, int nf, const char * name) {
    auto S = [&](int i) -> ggml_tensor * { return (i < nsrc && src[i] >= 0) ? c->t[src[i]] : nullptr; };
    auto I = [&](int i) -> int64_t { return i < ni ? ia[i] : 0; };
    auto F = [&](int i) -> float { return i < nf ? fa[i] : 0.0f; };
    ggml_context * g = c->ctx;
    std::string o(op);
    ggml_tensor * r = nullptr;
    if      (o == "mul_mat")   r = ggml_mul_mat(g, S(0), S(1));
    else if (o == "add")       r = ggml_add(g, S(0), S(1));
    else if (o == "sub")       r = ggml_sub(g, S(0), S(1));
    else if (o == "mul")       r = ggml_mul(g, S(0), S(1));
    else if (o == "div")       r = ggml_div(g, S(0), S(1));
    else if (o == "rms_norm")  r = ggml_rms_norm(g, S(0), F(0));
    else if (o == "norm")      r = ggml_norm(g, S(0), F(0));
    else if (o == "unary")     r = ggml_unary(g, S(0), (ggml_unary_op)I(0));
    else if (o == "glu")       r = ggml_glu(g, S(0), (ggml_glu_op)I(0), I(1) != 0);
    else if (o == "glu_split") r = ggml_glu_split(g, S(0), S(1), (ggml_glu_op)I(0));
    else if (o == "scale")     r = ggml_scale_bias(g, S(0), F(0), F(1));
    else if (o == "sqr")       r = ggml_sqr(g, S(0));
    else if (o == "sqrt")      r = ggml_sqrt(g, S(0));
    else if (o == "sin")       r = ggml_sin(g, S(0));
    else if (o == "cos")       r = ggml_cos(g, S(0));
    else if (o == "log")       r = ggml_log(g, S(0));
    else if (o == "clamp")     r = ggml_clamp(g, S(0), F(0), F(1));
    else if (o == "leaky_relu") r = ggml_leaky_relu(g, S(0), F(0), false);
    else if (o == "fill")      r = ggml_fill(g, S(0), F(0));
    else if (o == "rope_ext")  r = ggml_rope_ext(g, S(0), S(1), S(2), (int)I(0), (int)I(1), (int)I(2),
                                                 F(0), F(1), F(2), F(3), F(4), F(5));
    else if (o == "soft_max_ext") r = ggml_soft_max_ext(g, S(0), S(1), F(0), F(1));
    else if (o == "get_rows")  r = ggml_get_rows(g, S(0), S(1));
    else if (o == "set_rows")  r = ggml_set_rows(g, S(0), S(1), S(2));
    else if (o == "cpy")       r = ggml_cpy(g, S(0), S(1));
    else if (o == "cast")      r = ggml_cast(g, S(0), (ggml_type)I(0));
    else if (o == "cont")      r = ggml_cont(g, S(0));
    else if (o == "dup")       r = ggml_dup(g, S(0));
    else if (o == "reshape")   r = ggml_reshape_4d(g, S(0), I(0), I(1), I(2), I(3));
    else if (o == "view")      r = ggml_view_4d(g, S(0), I(0), I(1), I(2), I(3), (size_t)I(4), (size_t)I(5),
                                                (size_t)I(6), (size_t)I(7));
    else if (o == "permute")   r = ggml_permute(g, S(0), (int)I(0), (int)I(1), (int)I(2), (int)I(3));
    else if (o == "transpose") r = ggml_transpose(g, S(0));
    else if (o == "flash_attn_ext") {
        r = ggml_flash_attn_ext(g, S(0), S(1), S(2), S(3), F(0), F(1), F(2));
        if (r && I(0)) ggml_flash_attn_ext_set_prec(r, (ggml_prec)I(0));
    }
    else if (o == "argmax")    r = ggml_argmax(g, S(0));
    else if (o == "concat")    r = ggml_concat(g, S(0), S(1), (int)I(0));
    else if (o == "repeat")    r = ggml_repeat(g, S(0), S(1));
    else if (o == "sum_rows")  r = ggml_sum_rows(g, S(0));
    else if (o == "mean")      r = ggml_mean(g, S(0));
    else if (o == "arange")    r = ggml_arange(g, F(0), F(1), F(2));
    else if (o == "cumsum")    r = ggml_cumsum(g, S(0));
    else if (o == "im2col")    r = ggml_im2col(g, S(0), S(1), (int)I(0), (int)I(1), (int)I(2), (int)I(3), (int)I(4), (int)I(5), I(6) != 0,
                                               (ggml_type)I(7));
    else if (o == "interpolate") r = ggml_interpolate(g, S(0), I(0), I(1), I(2), I(3), (uint32_t)I(4));
    else if (o == "pool_2d")   r = ggml_pool_2d(g, S(0), (ggml_op_pool)I(0), (int)I(1), (int)I(2), (int)I(3), (int)I(4), F(0), F(1));
    else if (o == "conv_2d_dw") r = ggml_conv_2d_dw_direct(g, S(0), S(1), (int)I(0), (int)I(1), (int)I(2), (int)I(3), (int)I(4), (int)I(5));
    else if (o == "pad_ext")   r = ggml_pad_ext(g, S(0), (int)I(0), (int)I(1), (int)I(2), (int)I(3), (int)I(4), (int)I(5), (int)I(6), (int)I(7));
    else if (o == "pad_reflect_1d") r = ggml_pad_reflect_1d(g, S(0), (int)I(0), (int)I(1));
    else if (o == "custom") {
        // The paged nodes of scheme/core.ss:222-271: no function, userdata = packed u64.
        ggml_tensor * args[GGML_MAX_SRC] = {};
        for (int i = 0; i < nsrc; i++) args[i] = S(i);
        r = ggml_custom_4d(g, (ggml_type)I(0), I(1), I(2), I(3), I(4), args, nsrc, nullptr, 1,
                           (void *)(uintptr_t)(uint64_t)I(5));
    } else {
        c->err = "tlref_op: unknown op " + o;
        return -1;
    }
    if (r && name && name[0]) ggml_set_name(r, name);
    return push(c, r);
}

static int find(tlref_ctx * c, const ggml_tensor * x) {
    if (!x) return -1;
    for (size_t i = 0; i < c->t.size(); i++) if (c->t[i] == x) return (int)i;
    return -2;
}

// Metadata in the order native_ir.rs copies it into the IR.
void tlref_info(tlref_ctx * c, int id, int * type, int64_t * ne, uint64_t * nb, char * opname /*32*/,
                int32_t * op_params /*16*/, int * src /*10*/, int * view_src, uint64_t * view_offs) {
    const ggml_tensor * x = c->t[id];
    *type = (int)x->type;
    for (int i = 0; i < 4; i++) { ne[i] = x->ne[i]; nb[i] = x->nb[i]; }
    snprintf(opname, 32, "%s", ggml_op_name(x->op));
    memcpy(op_params, x->op_params, 16 * sizeof(int32_t));
    for (int i = 0; i < GGML_MAX_SRC && i < 10; i++) src[i] = find(c, x->src[i]);
    *view_src = find(c, x->view_src);
    *view_offs = x->view_offs;
}

// Builds the forward graph of `outs` and computes it on the CPU backend.
// Returns 0 on success; *ms receives the wall time of the compute call alone.
int tlref_compute(tlref_ctx * c, const int * outs, int nouts, int repeat, double * ms) {
    ggml_cgraph * gf = ggml_new_graph_custom(c->ctx, 16384, false);
    for (int i = 0; i < nouts; i++) ggml_build_forward_expand(gf, c->t[outs[i]]);
    if (!c->cpu) {
        c->cpu = ggml_backend_cpu_init();
        if (!c->cpu) { c->err = "no cpu backend"; return -1; }
        ggml_backend_cpu_set_n_threads(c->cpu, c->n_threads);
    }
    double best = 1e30;
    for (int r = 0; r < (repeat > 0 ? repeat : 1); r++) {
        int64_t t0 = ggml_time_us();
        ggml_status st = ggml_backend_graph_compute(c->cpu, gf);
        int64_t t1 = ggml_time_us();
        if (st != GGML_STATUS_SUCCESS) { c->err = "graph compute failed"; return -2; }
        double d = (t1 - t0) / 1000.0;
        if (d < best) best = d;
    }
    if (ms) *ms = best;
    return ggml_graph_n_nodes(gf);
}

const char * tlref_build_flags(void) {
#ifdef TLREF_FLAGS
    return TLREF_FLAGS;
#else
    return "";
#endif
}


// What the reference's own GGUF reader (vendored gguf.cpp, the one gguf.rs wraps) sees in a file: one line
// per key and per tensor. Returns the text length, or -1 when the file does not parse.
int64_t tlref_gguf_summary(const char * path, char * out, int64_t cap) {
    struct gguf_init_params ip = { /*no_alloc*/ true, /*ctx*/ nullptr };
    struct gguf_context * g = gguf_init_from_file(path, ip);
    if (!g) return -1;
    std::string t;
    char line[512];
    snprintf(line, sizeof line, "version %u alignment %zu data_offset %zu\n", gguf_get_version(g), gguf_get_alignment(g), gguf_get_data_offset(g));
    t += line;
    const int64_t nkv = gguf_get_n_kv(g);
    for (int64_t i = 0; i < nkv; i++) {
        const enum gguf_type ty = gguf_get_kv_type(g, i);
        if (ty == GGUF_TYPE_STRING) snprintf(line, sizeof line, "kv %s string %s\n", gguf_get_key(g, i), gguf_get_val_str(g, i));
        else if (ty == GGUF_TYPE_UINT32) snprintf(line, sizeof line, "kv %s u32 %u\n", gguf_get_key(g, i), gguf_get_val_u32(g, i));
        else if (ty == GGUF_TYPE_ARRAY) snprintf(line, sizeof line, "kv %s array %d %zu\n", gguf_get_key(g, i), (int)gguf_get_arr_type(g, i), gguf_get_arr_n(g, i));
        else snprintf(line, sizeof line, "kv %s type %d\n", gguf_get_key(g, i), (int)ty);
        t += line;
    }
    const int64_t nt = gguf_get_n_tensors(g);
    for (int64_t i = 0; i < nt; i++) {
        snprintf(line, sizeof line, "tensor %s type %d offset %zu size %zu\n", gguf_get_tensor_name(g, i), (int)gguf_get_tensor_type(g, i),
                 gguf_get_tensor_offset(g, i), gguf_get_tensor_size(g, i));
        t += line;
    }
    gguf_free(g);
    if ((int64_t)t.size() + 1 > cap) return -1;
    memcpy(out, t.c_str(), t.size() + 1);
    return (int64_t)t.size();
}

}  // extern "C"
