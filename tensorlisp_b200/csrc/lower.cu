// Lowers graph nodes to launches, by ggml op name (reference: crates/kernels/src/cuda/lower.rs:177-213),
// after a few IR rewrites that form the fused ops of a decoder step (reference: the fusion rules of
// crates/kernels/src/vulkan/fuse.rs:56-152, which its CUDA executor does not apply).
#include <cmath>
#include <cstdlib>
#include <map>

#include "kernels.h"
#include "tlb_internal.h"

namespace tlb {

namespace {

[[noreturn]] void unsupported(const Tensor &t, const std::string &why) { throw Unsupported{t.op, t.name, why}; }

bool plain(uint32_t ty) { return ty == 0 || ty == 1 || ty == 30 || ty == 26 || ty == 27; }
bool gemv_type(uint32_t ty) { return ty == TLB_TYPE_Q8_0 || ty == TLB_TYPE_Q4_0 || ty == TLB_TYPE_Q4_K; }
// block types that are read through the element decoders only (dequant.cuh): rows for GET_ROWS / CPY, weights of the
// generic mul_mat (decoded weights times f32 activations)
bool decoded_type(uint32_t ty) {
    return ty == TLB_TYPE_Q4_1 || ty == TLB_TYPE_Q5_0 || ty == TLB_TYPE_Q5_1 || ty == TLB_TYPE_Q2_K || ty == TLB_TYPE_Q3_K || ty == TLB_TYPE_Q5_K ||
           ty == TLB_TYPE_Q6_K;
}
bool mm_weight_ok(uint32_t ty) { return ty == 0 || ty == 1 || ty == 30 || gemv_type(ty) || decoded_type(ty); }

TView view_of(const Tensor &t) {
    TView v;
    for (int i = 0; i < 4; i++) {
        v.ne[i] = t.ne[i];
        v.nb[i] = (int64_t)t.nb[i];
    }
    return v;
}

// tensor-core mul_mat kernels by weight type
bool tc_supported(uint32_t wty, int64_t K, int64_t M, int64_t N) {
    if (wty == TLB_TYPE_Q4_K) return mmq_tc_supported(wty, K, M, N);
    if (wty == TLB_TYPE_Q8_0) return tc_available() && mmq_tc8_supported(K, M, N);
    return false;
}
TcPlan tc_plan(uint32_t wty, int64_t K, int64_t M, int64_t N, int sm) {
    return wty == TLB_TYPE_Q8_0 ? mmq_tc8_plan(K, M, N, sm) : mmq_tc_plan(K, M, N, sm);
}

int act_kind_for(uint32_t wty) { return wty == TLB_TYPE_Q4_K ? ACT_Q8_K : ACT_Q8_0; }
bool is_qact(const std::string &op) { return op == "QUANT_ACT" || op == "ROW_QUANT"; }

struct L {
    const LowerCtx &c;
    int32_t id;
    int pos;
    std::vector<Dispatch> &out;
    const Tensor &t() const { return c.g->tensors[id]; }
    const Tensor &T(int32_t i) const { return c.g->tensors[i]; }
    Place place(int32_t i) const { return c.layout->place[i]; }
    int32_t src(int i) const {
        const int32_t s = t().src[i];
        if (s < 0) throw std::string(t().op + " `" + t().name + "` is missing source " + std::to_string(i));
        return s;
    }
    void push(std::function<cudaError_t(const RunCtx &)> fn) { out.push_back({t().op + " " + t().name, std::move(fn)}); }
    void need_plain(std::initializer_list<int32_t> ids) const {
        for (int32_t s : ids)
            if (!plain(T(s).ty)) unsupported(t(), "quantized operand");
    }
    void need_f32(std::initializer_list<int32_t> ids) const {
        for (int32_t s : ids)
            if (T(s).ty != TLB_TYPE_F32) unsupported(t(), "operands must be f32");
    }
};

void lower_bin(L &l) {
    const int32_t a = l.src(0), b = l.src(1);
    l.need_f32({a, b, l.id});
    BinArgs p{view_of(l.T(a)), view_of(l.T(b)), view_of(l.t()), 0};
    const std::string &op = l.t().op;
    p.op = op == "ADD" ? 0 : op == "SUB" ? 1 : op == "MUL" ? 2 : 3;
    for (int i = 0; i < 4; i++)
        if (p.b.ne[i] == 0 || p.d.ne[i] % p.b.ne[i] != 0) unsupported(l.t(), "the second operand does not broadcast into the first");
    const Place pa = l.place(a), pb = l.place(b), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_bin(p, r.at(pa), r.at(pb), r.at(pd), r.stream); });
}

void lower_unary(L &l) {
    const int32_t a = l.src(0);
    const Tensor &t = l.t();
    l.need_plain({a, l.id});
    UnaryArgs p{view_of(l.T(a)), view_of(t), 0, 0.f, 0.f, l.T(a).ty, t.ty};
    const std::string &op = t.op;
    if (op == "SCALE") { p.code = 100; p.p0 = t.param_f32(0); p.p1 = t.param_f32(1); }
    else if (op == "FILL") { p.code = 101; p.p0 = t.param_f32(0); }
    else if (op == "CLAMP") { p.code = 102; p.p0 = t.param_f32(0); p.p1 = t.param_f32(1); }
    else if (op == "LEAKY_RELU") { p.code = 103; p.p0 = t.param_f32(0); }
    else if (op == "SQR") p.code = 104;
    else if (op == "SQRT") p.code = 105;
    else if (op == "SIN") p.code = 106;
    else if (op == "COS") p.code = 107;
    else if (op == "LOG") p.code = 108;
    else {
        const int n = t.op_params[0];
        if (n == 17) unsupported(t, "xielu");
        if (n < 0 || n > 21) unsupported(t, "unary op " + std::to_string(n));
        p.code = n;
    }
    if (l.T(a).nelements() != t.nelements()) unsupported(t, "source and destination differ in size");
    const Place pa = l.place(a), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_unary(p, r.at(pa), r.at(pd), r.stream); });
}

void lower_glu(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0);
    const int32_t b = t.src[1];
    const int glu_op = t.op_params[0];
    const bool swapped = t.op_params[1] != 0;
    if (!(glu_op == 0 || glu_op == 1 || glu_op == 2 || glu_op == 4 || glu_op == 5)) unsupported(t, "glu op " + std::to_string(glu_op));
    l.need_f32({a, l.id});
    const Tensor &ta = l.T(a);
    if (ta.nb[0] != 4 || !t.is_contiguous()) unsupported(t, "needs dense rows");
    GluArgs p;
    p.n = t.ne[0];
    p.rows = t.nrows();
    p.glu_op = glu_op;
    if (!ta.is_contiguous_n(1) && ta.nrows() != ta.ne[1]) unsupported(t, "needs uniformly strided rows");
    p.lda = (int64_t)ta.nb[1] / 4;
    int64_t a_off = 0, b_off = 0;
    Place pb;
    if (b >= 0) {
        const Tensor &tb = l.T(b);
        l.need_f32({b});
        if (tb.nb[0] != 4 || tb.ne[0] != t.ne[0] || tb.nrows() != t.nrows()) unsupported(t, "operands differ in shape");
        p.ldb = (int64_t)tb.nb[1] / 4;
        pb = l.place(b);
    } else {
        if (ta.ne[0] != 2 * t.ne[0]) unsupported(t, "unsplit glu takes a source twice as wide");
        p.ldb = p.lda;
        pb = l.place(a);
        a_off = swapped ? t.ne[0] * 4 : 0;
        b_off = swapped ? 0 : t.ne[0] * 4;
    }
    if (ta.nrows() > 1 && (ta.ne[2] > 1 || ta.ne[3] > 1) && !ta.is_contiguous_n(1)) unsupported(t, "needs uniformly strided rows");
    const Place pa = l.place(a), pd = l.place(l.id);
    l.push([=](const RunCtx &r) {
        return launch_glu(p, (const float *)(r.at(pa) + a_off), (const float *)(r.at(pb) + b_off), (float *)r.at(pd), r.stream);
    });
}

void lower_norm(L &l, bool fused_mul) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0);
    l.need_f32({a, l.id});
    if (l.T(a).nb[0] != 4 || t.nb[0] != 4) unsupported(t, "needs dense rows");
    NormArgs p;
    p.a = view_of(l.T(a));
    p.d = view_of(t);
    p.rms = (t.op == "RMS_NORM" || t.op == "RMS_NORM_MUL") ? 1 : 0;
    p.eps = t.param_f32(fused_mul ? 15 : 0);
    p.has_w = fused_mul ? 1 : 0;
    Place pw;
    if (fused_mul) {
        const int32_t w = l.src(1);
        p.w = view_of(l.T(w));
        pw = l.place(w);
    } else {
        p.w = p.a;
    }
    const Place pa = l.place(a), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_norm(p, r.at(pa), fused_mul ? r.at(pw) : nullptr, r.at(pd), r.stream); });
}

// rope parameters of a ROPE node (or of a node that carries a copy of them)
RopeArgs rope_params(const Tensor &t, int64_t row_len) {
    RopeArgs p{};
    p.n_dims = t.op_params[1];
    p.mode = t.op_params[2];
    if (p.mode != 0 && p.mode != 2) unsupported(t, "only normal and neox rope (mrope/vision are not supported)");
    const float freq_base = t.param_f32(5);
    p.freq_scale = t.param_f32(6);
    p.ext_factor = t.param_f32(7);
    p.attn_factor = t.param_f32(8);
    const float beta_fast = t.param_f32(9), beta_slow = t.param_f32(10);
    const float n_ctx_orig = (float)t.op_params[4];
    if (p.n_dims <= 0 || p.n_dims > row_len || p.n_dims % 2) unsupported(t, "bad n_dims");
    p.theta_scale = powf(freq_base, -2.0f / (float)p.n_dims);
    // ggml_rope_yarn_corr_dims (ggml.c:4369-4381)
    auto corr = [&](float beta) { return (float)p.n_dims * logf(n_ctx_orig / (beta * 2.0f * (float)M_PI)) / (2.0f * logf(freq_base)); };
    p.corr0 = fmaxf(0.f, floorf(corr(beta_fast)));
    p.corr1 = fminf((float)p.n_dims - 1.f, ceilf(corr(beta_slow)));
    return p;
}

void lower_rope(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0), pos = l.src(1);
    const int32_t ff = t.src[2];
    if (l.T(pos).ty != TLB_TYPE_I32 || l.T(pos).ne[0] != l.T(a).ne[2]) unsupported(t, "needs one i32 position per token");
    if (ff >= 0 && (l.T(ff).ty != TLB_TYPE_F32 || l.T(ff).nb[0] != 4)) unsupported(t, "frequency factors must be f32");
    const uint32_t aty = l.T(a).ty, dty = t.ty;
    if (!(aty == 0 || aty == 1) || !(dty == 0 || dty == 1)) unsupported(t, "rope takes f32 or f16");
    RopeArgs p = rope_params(t, t.ne[0]);
    p.a = view_of(l.T(a));
    p.d = view_of(t);
    p.aty = aty;
    p.dty = dty;
    p.has_ff = ff >= 0;
    const Place pa = l.place(a), pp = l.place(pos), pd = l.place(l.id);
    Place pf;
    if (ff >= 0) pf = l.place(ff);
    const bool hf = ff >= 0;
    l.push([=](const RunCtx &r) {
        return launch_rope(p, r.at(pa), (const int32_t *)r.at(pp), hf ? (const float *)r.at(pf) : nullptr, r.at(pd), r.stream);
    });
}

// ROPE_KV_WRITE (pseudo-op made by fuse_rope_cache): src = q, k, v (f32), pos, freq factors or -1,
// key pool, value pool, slots, and the f16 query it produces. op_params: the rope's, with the
// kv-head count and block size in [12], [13].
void lower_rope_kv(L &l) {
    const Tensor &t = l.t();
    const int32_t q = l.src(0), k = l.src(1), v = l.src(2), pos = l.src(3), kc = l.src(5), vc = l.src(6), slots = l.src(7), q16 = l.src(8);
    const int32_t ff = t.src[4];
    const Tensor &tq = l.T(q), &tk = l.T(k), &tv = l.T(v);
    RopeKvArgs p{};
    p.rope = rope_params(t, tq.ne[0]);
    p.rope.a = view_of(tq);
    p.rope.has_ff = ff >= 0;
    p.k = view_of(tk);
    p.hs = (int)tq.ne[0];
    p.heads = (int)tq.ne[1];
    p.tokens = (int)tq.ne[2];
    p.kv_heads = t.op_params[12];
    p.block_size = t.op_params[13];
    if (p.block_size < 1) unsupported(t, "the block size of a cache write must be at least 1");
    p.pool_slots = l.T(kc).nelements() / ((int64_t)p.kv_heads * p.hs);
    // v arrives as [hs * kv_heads, tokens]
    p.v = view_of(tv);
    p.v.nb[2] = (int64_t)tv.nb[1];
    p.v.nb[1] = (int64_t)p.hs * 4;
    const Place pq = l.place(q), pk = l.place(k), pv = l.place(v), pp = l.place(pos), pkc = l.place(kc), pvc = l.place(vc),
                psl = l.place(slots), pq16 = l.place(q16);
    Place pf;
    if (ff >= 0) pf = l.place(ff);
    const bool hf = ff >= 0;
    l.push([=](const RunCtx &r) {
        return launch_rope_kv(p, r.at(pq), r.at(pk), r.at(pv), (const int32_t *)r.at(pp), hf ? (const float *)r.at(pf) : nullptr,
                              r.at(pq16), r.at(pkc), r.at(pvc), (const int64_t *)r.at(psl), r.err, r.stream);
    });
}

void lower_soft_max(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0);
    if (t.src[2] >= 0) unsupported(t, "sinks are not supported by the soft_max lowering");
    l.need_f32({a, l.id});
    const int32_t m = t.src[1];
    if (m >= 0 && !(l.T(m).ty == 0 || l.T(m).ty == 1)) unsupported(t, "mask must be f16 or f32");
    if (l.T(a).nb[0] != 4 || t.nb[0] != 4) unsupported(t, "needs dense rows");
    SoftmaxArgs p;
    p.a = view_of(l.T(a));
    p.d = view_of(t);
    p.has_mask = m >= 0;
    p.m = m >= 0 ? view_of(l.T(m)) : p.a;
    p.mty = m >= 0 ? l.T(m).ty : 0;
    p.scale = t.param_f32(0);
    p.max_bias = t.param_f32(1);
    p.n_head_log2 = 1 << (int)floorf(log2f((float)l.T(a).ne[2]));
    p.m0 = powf(2.0f, -p.max_bias / (float)p.n_head_log2);
    p.m1 = powf(2.0f, -(p.max_bias / 2.0f) / (float)p.n_head_log2);
    const Place pa = l.place(a), pd = l.place(l.id);
    Place pm;
    if (m >= 0) pm = l.place(m);
    const bool hm = m >= 0;
    l.push([=](const RunCtx &r) { return launch_soft_max(p, r.at(pa), hm ? r.at(pm) : nullptr, r.at(pd), r.stream); });
}

void lower_get_rows(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0), ids = l.src(1);
    const uint32_t aty = l.T(a).ty;
    if (!(plain(aty) || gemv_type(aty) || decoded_type(aty))) unsupported(t, std::string("rows of ggml type ") + type_traits(aty)->name);
    if (!(l.T(ids).ty == 26 || l.T(ids).ty == 27)) unsupported(t, "row indices must be i32 or i64");
    if (!plain(t.ty)) unsupported(t, "operand type");
    RowsArgs p{view_of(l.T(a)), view_of(l.T(ids)), view_of(t), aty, l.T(ids).ty, t.ty};
    const Place pa = l.place(a), pi = l.place(ids), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_get_rows(p, r.at(pa), r.at(pi), r.at(pd), r.stream); });
}

void lower_set_rows(L &l) {
    // ggml_set_rows(a = destination, b = rows, c = ids): the node is a view of a with src[0] = b, src[1] = c
    const Tensor &t = l.t();
    const int32_t rows = l.src(0), ids = l.src(1);
    l.need_plain({rows, l.id});
    if (!(l.T(ids).ty == 26 || l.T(ids).ty == 27)) unsupported(t, "row indices must be i32 or i64");
    if (l.T(rows).ne[0] != t.ne[0]) unsupported(t, "rows and destination differ in width");
    RowsArgs p{view_of(l.T(rows)), view_of(l.T(ids)), view_of(t), l.T(rows).ty, l.T(ids).ty, t.ty};
    const Place pa = l.place(rows), pi = l.place(ids), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_set_rows(p, r.at(pa), r.at(pi), r.at(pd), r.stream); });
}

void lower_cpy(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0);
    const Tensor &ta = l.T(a);
    if (ta.nelements() != t.nelements()) unsupported(t, "source and destination differ in size");
    if (!(plain(ta.ty) || gemv_type(ta.ty) || decoded_type(ta.ty))) unsupported(t, "operand type");
    if (!plain(t.ty)) unsupported(t, "operand type");
    CpyArgs p{view_of(ta), view_of(t), ta.ty, t.ty};
    const Place pa = l.place(a), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_cpy(p, r.at(pa), r.at(pd), r.stream); });
}

void lower_argmax(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0);
    l.need_f32({a});
    if (t.ty != TLB_TYPE_I32) unsupported(t, "argmax writes i32");
    if (l.T(a).nb[0] != 4) unsupported(t, "needs dense rows");
    if (!l.T(a).is_contiguous_n(1) ) unsupported(t, "needs uniformly strided rows");
    const TView v = view_of(l.T(a));
    const Place pa = l.place(a), pd = l.place(l.id);
    l.push([=](const RunCtx &r) { return launch_argmax(v, r.at(pa), (int32_t *)r.at(pd), r.stream); });
}

void lower_simple(L &l) {
    const Tensor &t = l.t();
    SimpleArgs p{};
    p.d = view_of(t);
    const Place pd = l.place(l.id);
    if (t.op == "ARANGE") {
        if (t.ty != 0) unsupported(t, "arange writes f32");
        p.f0 = t.param_f32(0);
        p.f1 = t.param_f32(2);
        l.push([=](const RunCtx &r) { return launch_arange(p, r.at(pd), r.stream); });
        return;
    }
    const int32_t a = l.src(0);
    l.need_f32({a, l.id});
    p.a = view_of(l.T(a));
    const Place pa = l.place(a);
    if (t.op == "CONCAT") {
        const int32_t b = l.src(1);
        l.need_f32({b});
        p.b = view_of(l.T(b));
        p.i0 = t.op_params[0];
        if (p.i0 < 0 || p.i0 > 3) unsupported(t, "bad concat dimension");
        const Place pb = l.place(b);
        l.push([=](const RunCtx &r) { return launch_concat(p, r.at(pa), r.at(pb), r.at(pd), r.stream); });
    } else if (t.op == "REPEAT") {
        l.push([=](const RunCtx &r) { return launch_repeat(p, r.at(pa), r.at(pd), r.stream); });
    } else {  // SUM_ROWS / MEAN
        if (l.T(a).nb[0] != 4) unsupported(t, "needs dense rows");
        p.i0 = t.op == "MEAN";
        l.push([=](const RunCtx &r) { return launch_sum_rows(p, r.at(pa), r.at(pd), r.stream); });
    }
}

// the node after this one is an ALLREDUCE of this node's result
bool allreduce_follows(const L &l) {
    const Graph &g = *l.c.g;
    if (getenv("TLB_SPLITK_REDUCE_LAUNCH")) return false;   // keep the separate launch that adds the partial sums
    if ((size_t)l.pos + 1 >= g.nodes.size()) return false;
    const Tensor &nx = g.tensors[g.nodes[l.pos + 1]];
    return nx.op == "ALLREDUCE" && nx.src[0] == l.id;
}

// ---- MUL_MAT (lower.rs:543-571). Quantized weights take int8 activations quantized once per
// distinct activation tensor by a QUANT_ACT node that rewrite_graph put in src[2].
void lower_mul_mat(L &l) {
    const Tensor &t = l.t();
    const int32_t w = l.src(0), x = l.src(1);
    const Tensor &tw = l.T(w), &tx = l.T(x);
    if (!mm_weight_ok(tw.ty)) unsupported(t, std::string("weights of ggml type ") + type_traits(tw.ty)->name);
    if (tx.ty != TLB_TYPE_F32) unsupported(t, "activations must be f32");
    if (t.ty != TLB_TYPE_F32) unsupported(t, "the result must be f32");
    if (tw.ne[0] != tx.ne[0] || t.ne[0] != tw.ne[1] || t.ne[1] != tx.ne[1] || tw.ne[2] == 0 || tw.ne[3] == 0 ||
        t.ne[2] != tx.ne[2] || t.ne[3] != tx.ne[3] || t.ne[2] % tw.ne[2] != 0 || t.ne[3] % tw.ne[3] != 0)
        unsupported(t, "inconsistent shapes");
    if (tw.nb[0] != type_traits(tw.ty)->size) unsupported(t, "weight rows must be dense");
    const Place pw = l.place(w), px = l.place(x), pd = l.place(l.id);
    const int64_t K = tw.ne[0], M = tw.ne[1], N = tx.ne[1];
    const int sm = l.c.dev->prop.multiProcessorCount;
    MMGeneric g{};
    g.wtype = tw.ty;
    g.w = view_of(tw);
    g.x = view_of(tx);
    g.y = view_of(t);
    g.r2 = t.ne[2] / tw.ne[2];
    g.r3 = t.ne[3] / tw.ne[3];
    if (!gemv_type(tw.ty)) {
        l.push([=](const RunCtx &r) { return launch_mm_generic(g, r.at(pw), r.at(px), r.at(pd), r.stream); });
        return;
    }
    const int32_t qa = t.src[2];
    if (qa < 0 || !is_qact(l.T(qa).op)) unsupported(t, "activations could not be quantized (rows must be dense f32 with uniformly strided columns and a length that is a multiple of the block size)");
    const Place pq = l.place(qa);
    const ActLayout a = act_layout(act_kind_for(tw.ty), K, tx.nrows());
    const bool batched = tw.ne[2] * tw.ne[3] * t.ne[2] * t.ne[3] != 1;
    const bool dense_w = tw.nb[1] == tw.row_size();
    const bool dense_y = t.is_contiguous();
    if (!batched && dense_w && dense_y && l.T(qa).op_params[1] > 0 && tc_supported(tw.ty, K, M, N) && !getenv("TLB_MM_GENERIC") &&
        !getenv("TLB_NO_TC")) {
        // tensor-core path: the QUANT_ACT node also packed the activations into per-super-block blobs
        const TcPlan tp = tc_plan(tw.ty, K, M, N, sm);
        if (tp.npad != l.T(qa).op_params[1]) throw std::string("activation blobs were packed for another column count");
        const int64_t sc = l.c.layout->scratch[l.pos];
        if (tp.partial_bytes > 0 && sc < 0) throw std::string("split-K scratch was not planned");
        Place ps;
        ps.buf = BUF_ARENA;
        ps.off = sc < 0 ? 0 : (uint64_t)sc;
        const uint64_t blob_off = a.bytes;
        const bool q8 = tw.ty == TLB_TYPE_Q8_0;
        // a row-parallel projection: when the exchange that follows runs over peer memory, it adds the K-split
        // partial sums itself (decided at launch: the communicator may be set up after the program is compiled)
        const bool ar_next = !q8 && tp.n_split > 1 && tp.n_col_chunks == 1 && allreduce_follows(l);
        tlb_device *dev = l.c.dev;
        const size_t n_out = (size_t)(N * M);
        l.push([=](const RunCtx &r) {
            const bool leave = ar_next && comm_p2p_takes(dev, n_out);
            return q8 ? launch_mmq_tc8(tp, r.at(pw), K, M, N, r.at(pq) + blob_off, (float *)r.at(pd), M, r.at(ps), r.err, r.stream)
                      : launch_mmq_tc(tp, r.at(pw), K, M, N, r.at(pq) + blob_off, (float *)r.at(pd), M, r.at(ps), r.err, r.stream, leave);
        });
        return;
    }
    if (!batched && dense_w && dense_y && gemv_supported(tw.ty, K, M, N) && !getenv("TLB_MM_GENERIC")) {
        const uint32_t wty = tw.ty;
        l.push([=](const RunCtx &r) {
            return launch_gemv(wty, r.at(pw), K, M, a, r.at(pq), (float *)r.at(pd), M, sm, r.err, r.stream);
        });
        return;
    }
    g.a = a;
    l.push([=](const RunCtx &r) {
        MMGeneric gg = g;
        gg.act = r.at(pq);
        return launch_mm_generic(gg, r.at(pw), r.at(px), r.at(pd), r.stream);
    });
}

// MUL_MAT_GROUP (pseudo-op made by fuse_mul_mat_groups): up to three Q4_K mul_mats over the same
// activations (wq / wk / wv) in one tensor-core launch. src = w0, x, quantized x, w1, y1, w2, y2; the
// node's own tensor is y0.
void lower_mul_mat_group(L &l) {
    const Tensor &t = l.t();
    const int32_t x = l.src(1), qa = l.src(2);
    const Tensor &tx = l.T(x);
    const int64_t K = tx.ne[0], N = tx.ne[1];
    int n_mats = 0;
    Place pw[3], py[3];
    int64_t Ms[3] = {0, 0, 0}, Msum = 0;
    const int wslot[3] = {0, 3, 5}, yslot[3] = {-1, 4, 6};
    for (int j = 0; j < 3; j++) {
        if (t.src[wslot[j]] < 0) break;
        const int32_t w = t.src[wslot[j]], y = j == 0 ? l.id : l.src(yslot[j]);
        const Tensor &tw = l.T(w), &ty = l.T(y);
        if (tw.ty != TLB_TYPE_Q4_K || tw.ne[0] != K || tw.nb[1] != tw.row_size() || ty.ty != TLB_TYPE_F32 || !ty.is_contiguous() ||
            ty.ne[0] != tw.ne[1] || ty.ne[1] != N)
            throw std::string("a grouped mul_mat lost its shape invariants");
        pw[j] = l.place(w);
        py[j] = l.place(y);
        Ms[j] = tw.ne[1];
        Msum += Ms[j];
        n_mats++;
    }
    const int sm = l.c.dev->prop.multiProcessorCount;
    const TcPlan tp = mmq_tc_plan(K, Msum, N, sm);
    if (tp.npad != l.T(qa).op_params[1] || tp.n_col_chunks != 1) throw std::string("activation blobs were packed for another column count");
    const ActLayout a = act_layout(ACT_Q8_K, K, tx.nrows());
    const int64_t sc = l.c.layout->scratch[l.pos];
    if (tp.partial_bytes > 0 && sc < 0) throw std::string("split-K scratch was not planned");
    Place ps;
    ps.buf = BUF_ARENA;
    ps.off = sc < 0 ? 0 : (uint64_t)sc;
    const Place pq = l.place(qa);
    const uint64_t blob_off = a.bytes;
    l.push([=](const RunCtx &r) {
        const void *W[3] = {nullptr, nullptr, nullptr};
        float *Y[3] = {nullptr, nullptr, nullptr};
        for (int j = 0; j < n_mats; j++) {
            W[j] = r.at(pw[j]);
            Y[j] = (float *)r.at(py[j]);
        }
        return launch_mmq_tc_group(tp, n_mats, W, K, Ms, N, r.at(pq) + blob_off, Y, Ms[0], r.at(ps), r.err, r.stream);
    });
}

void lower_quant_act(L &l) {
    const Tensor &t = l.t();
    const int32_t x = l.src(0);
    const Tensor &tx = l.T(x);
    const ActLayout a = act_layout(t.op_params[0], tx.ne[0], tx.nrows());
    const int64_t ldx = tx.nrows() > 1 ? (int64_t)tx.nb[1] / 4 : tx.ne[0];
    const Place px = l.place(x), pd = l.place(l.id);
    const int npad = t.op_params[1];   // > 0: also pack the blobs of the tensor-core path behind the Q8_K block
    if (a.kind == ACT_Q8_0 && npad == 256 && row_quant_q80_supported(a.K, RQ_PLAIN) && tx.nb[0] == 4 && ldx % 4 == 0) {
        // the prompt mul_mat reads the packed f16 operand only: one launch from the f32 rows straight to it
        RowQuantArgs p{};
        p.mode = RQ_PLAIN;
        p.K = a.K;
        p.N = a.N;
        p.lda = ldx;
        p.npad = npad;
        p.q80 = 1;
        p.qs_off = a.qs_off;
        p.d_off = a.d_off;
        p.blob_off = a.bytes;
        l.push([=](const RunCtx &r) {
            RowQuantArgs q = p;
            q.a = (const float *)r.at(px);
            q.out = r.at(pd);
            return launch_row_quant(q, r.stream);
        });
        return;
    }
    l.push([=](const RunCtx &r) {
        cudaError_t e = launch_act_quantize(a, (const float *)r.at(px), ldx, r.at(pd), r.stream);
        if (e == cudaSuccess && npad > 0)
            e = a.kind == ACT_Q8_0 ? launch_act_pack_tc8(a, r.at(pd), npad, r.at(pd) + a.bytes, r.stream)
                                   : launch_act_pack_tc(a, r.at(pd), npad, r.at(pd) + a.bytes, r.stream);
        return e;
    });
}

void partial_sums_in_front(const LowerCtx &c, int pos, int32_t mm_id, int &n_split, Place &ps);
bool exchange_fused_with_row_quant(const LowerCtx &c, int pos);

// ---- ROW_QUANT: a QUANT_ACT node that absorbed its producer (fuse_row_producers)
void lower_row_quant(L &l) {
    const Tensor &t = l.t();
    const int mode = t.op_params[2];
    const int32_t a = l.src(0);
    const Tensor &shape = mode == RQ_F16 ? l.T(l.src(5)) : l.T(a);
    RowQuantArgs p{};
    p.mode = mode;
    p.K = shape.ne[0];
    p.N = shape.nrows();
    const ActLayout al = act_layout(t.op_params[0] == ACT_Q8_0 ? ACT_Q8_0 : ACT_Q8_K, p.K, p.N);
    p.qs_off = al.qs_off;
    p.d_off = al.d_off;
    p.bsum_off = al.bsum_off;
    p.npad = t.op_params[1];
    p.blob_off = al.bytes;
    p.blob_bytes = p.npad > 0 ? mmq_tc_plan(p.K, 128, p.N, 148).blob_unit : 0;
    p.q80 = t.op_params[0] == ACT_Q8_0;
    p.eps = t.param_f32(15);
    p.lda = mode == RQ_F16 ? p.K : (p.N > 1 ? (int64_t)l.T(a).nb[1] / 4 : p.K);
    const int32_t b = t.src[1], w = t.src[3], sum = t.src[4];
    if (b >= 0) p.ldb = p.N > 1 ? (int64_t)l.T(b).nb[1] / 4 : p.K;
    if (w >= 0) p.wn = l.T(w).ne[0];
    if (sum >= 0) p.ld_sum = p.K;
    const Place pa = l.place(a), pd = l.place(l.id);
    Place pb, pw, ps;
    if (b >= 0) pb = l.place(b);
    if (w >= 0) pw = l.place(w);
    if (sum >= 0) ps = l.place(sum);
    // the all-reduce right in front may be folded into this launch (exchange_fused_with_row_quant)
    const bool fused_ar = l.pos > 0 && exchange_fused_with_row_quant(l.c, l.pos - 1);
    int ar_split = 0;
    Place par_data, par_part;
    tlb_device *dev = l.c.dev;
    if (fused_ar) {
        const int32_t ar = l.c.g->nodes[l.pos - 1];
        par_data = l.place(ar);
        partial_sums_in_front(l.c, l.pos - 1, l.T(ar).src[0], ar_split, par_part);
    }
    const size_t n_ar = (size_t)(p.N * p.K);
    l.push([=](const RunCtx &r) {
        RowQuantArgs q = p;
        q.a = (const float *)r.at(pa);
        q.b = b >= 0 ? (const float *)r.at(pb) : nullptr;
        q.w = w >= 0 ? (const float *)r.at(pw) : nullptr;
        q.sum_out = sum >= 0 ? (float *)r.at(ps) : nullptr;
        q.y_out = nullptr;
        q.out = r.at(pd);
        if (fused_ar && comm_p2p_takes(dev, n_ar))
            return comm_exchange_row_quant(dev, (float *)r.at(par_data), ar_split > 0 ? (const float *)r.at(par_part) : nullptr, ar_split, q,
                                           r.stream, r.err);
        return launch_row_quant(q, r.stream);
    });
}

// ---- CUSTOM: the paged nodes (lower.rs:660-759). userdata, low to high bits: kind (4), kv heads (4),
// block size (8), max context length (16), scale (f32).
struct PagedUd {
    int kind, kv_heads, block_size, max_ctx;
    float scale;
};
PagedUd paged_ud(const Tensor &t) {
    const uint64_t ud = (uint64_t)(uint32_t)t.op_params[4] | ((uint64_t)(uint32_t)t.op_params[5] << 32);
    PagedUd u;
    u.kind = (int)(ud & 15);
    u.kv_heads = (int)((ud >> 4) & 15);
    u.block_size = (int)((ud >> 8) & 255);
    u.max_ctx = (int)((ud >> 16) & 0xffff);
    const uint32_t bits = (uint32_t)(ud >> 32);
    std::memcpy(&u.scale, &bits, 4);
    return u;
}

bool paged_geom(const Graph &g, const Tensor &t, int sm, PagedGeom &pg) {
    const PagedUd u = paged_ud(t);
    if (u.kind != 1 || t.src[0] < 0 || t.src[3] < 0) return false;
    const Tensor &q = g.tensors[t.src[0]];
    pg.hs = (int)q.ne[0];
    pg.heads = (int)q.ne[1];
    pg.seqs = (int)q.ne[2];
    pg.kv_heads = u.kv_heads;
    pg.block_size = u.block_size;
    pg.max_ctx = u.max_ctx;
    pg.max_blocks = (int)g.tensors[t.src[3]].ne[0];
    pg.scale = u.scale;
    if (!paged_supported(pg)) return false;
    paged_plan(pg, sm);
    return true;
}

void lower_custom(L &l) {
    const Tensor &t = l.t();
    const PagedUd u = paged_ud(t);
    auto f16 = [&](int32_t s) { return l.T(s).ty == TLB_TYPE_F16; };
    if (u.kind == 1) {
        const int32_t q = l.src(0), kc = l.src(1), vc = l.src(2), tables = l.src(3), lens = l.src(4);
        const Tensor &tq = l.T(q);
        if (!(f16(q) && f16(kc) && f16(vc) && t.ty == TLB_TYPE_F16)) unsupported(t, "paged attention takes f16 q, caches and output");
        const uint64_t hs = (uint64_t)tq.ne[0], heads = (uint64_t)tq.ne[1];
        if (tq.nb[0] != 2 || tq.nb[1] != hs * 2 || tq.nb[2] != hs * heads * 2 || t.ne[0] != tq.ne[0] || t.ne[1] != tq.ne[1] || t.ne[2] != tq.ne[2] || !t.is_contiguous())
            unsupported(t, "paged attention takes a contiguous q and an output of its shape");
        if (l.T(tables).ty != TLB_TYPE_I32 || l.T(lens).ty != TLB_TYPE_I32 || !l.T(tables).is_contiguous() || !l.T(lens).is_contiguous())
            unsupported(t, "block tables and context lengths must be contiguous i32");
        if (l.T(tables).ne[1] != tq.ne[2] || l.T(lens).ne[0] != tq.ne[2]) unsupported(t, "one block-table row and one length per sequence");
        PagedGeom pg{};
        if (!paged_geom(*l.c.g, t, l.c.dev->prop.multiProcessorCount, pg))
            unsupported(t, "head size must be 64, 128 or 256 and the query heads a multiple of the kv heads");
        if ((int64_t)pg.max_blocks * pg.block_size < pg.max_ctx) unsupported(t, "block tables are shorter than the maximum context");
        const int64_t sc = l.c.layout->scratch[l.pos];
        if (paged_scratch_bytes(pg) > 0 && sc < 0) throw std::string("paged attention scratch was not planned");
        Place ps;
        ps.buf = BUF_ARENA;
        ps.off = sc < 0 ? 0 : (uint64_t)sc;
        const Place pq = l.place(q), pk = l.place(kc), pv = l.place(vc), pt = l.place(tables), pl = l.place(lens), pd = l.place(l.id);
        const int64_t pool_blocks = std::min(l.T(kc).nelements(), l.T(vc).nelements()) / ((int64_t)pg.kv_heads * pg.block_size * pg.hs);
        // src[9]: the Q8_K quantization of the output rows that fuse_attn_quant folded into this launch
        const int32_t qid = t.src[9];
        RowQuantArgs rq{};
        Place prq;
        if (qid >= 0) {
            if (pg.n_chunks != 1 || !paged_quant_fusable(pg)) throw std::string("the attention plan changed after its quantizer was folded in");
            rq.mode = RQ_F16;
            rq.K = (int64_t)pg.hs * pg.heads;
            rq.N = pg.seqs;
            const ActLayout al = act_layout(ACT_Q8_K, rq.K, rq.N);
            rq.qs_off = al.qs_off;
            rq.d_off = al.d_off;
            rq.bsum_off = al.bsum_off;
            rq.npad = l.T(qid).op_params[1];
            rq.blob_off = al.bytes;
            rq.blob_bytes = rq.npad > 0 ? mmq_tc_plan(rq.K, 128, rq.N, 148).blob_unit : 0;
            prq = l.place(qid);
        }
        l.push([=](const RunCtx &r) {
            RowQuantArgs a = rq;
            if (qid >= 0) a.out = r.at(prq);
            return launch_paged_attention(pg, r.at(pq), r.at(pk), r.at(pv), (const int32_t *)r.at(pt), (const int32_t *)r.at(pl),
                                          r.at(pd), r.at(ps), pool_blocks, r.err, r.stream, qid >= 0 ? &a : nullptr);
        });
    } else if (u.kind == 2) {
        const int32_t key = l.src(0), value = l.src(1), kc = l.src(2), vc = l.src(3), slots = l.src(4);
        const Tensor &tk = l.T(key);
        if (!(f16(key) && f16(value) && f16(kc) && f16(vc))) unsupported(t, "the cache write takes f16 keys, values and caches");
        const int tokens = (int)tk.nrows();
        if (l.T(slots).nelements() != 2 * (int64_t)tokens || tk.nb[1] != (uint64_t)tk.ne[0] * 2 || !tk.is_contiguous() || !l.T(value).is_contiguous() ||
            l.T(value).nelements() != tk.nelements())
            unsupported(t, "the cache write takes contiguous keys and one i64 slot per token");
        if (u.kv_heads < 1 || tk.ne[0] % u.kv_heads != 0 || (tk.ne[0] / u.kv_heads) % 8 != 0) unsupported(t, "head size must be a multiple of 8");
        const int hs = (int)(tk.ne[0] / u.kv_heads);
        if (u.block_size < 1) unsupported(t, "the block size of a cache write must be at least 1");
        const int64_t pool_slots = std::min(l.T(kc).nelements(), l.T(vc).nelements()) / ((int64_t)u.kv_heads * hs);
        const Place pk = l.place(key), pv = l.place(value), pkc = l.place(kc), pvc = l.place(vc), psl = l.place(slots);
        const int kvh = u.kv_heads, bs = u.block_size;
        l.push([=](const RunCtx &r) {
            return launch_cache_write(tokens, kvh, hs, bs, r.at(pk), r.at(pv), r.at(pkc), r.at(pvc), (const int64_t *)r.at(psl), pool_slots, r.err, r.stream);
        });
    } else {
        unsupported(t, "unknown custom op");
    }
}

// ---- FLASH_ATTN_EXT (lower.rs:575-657): dense attention, result [dv, heads, queries, batch] f32
// The kernel arguments of a node, or a reason why it is not supported
static const char *flash_args(const Graph &g, const Tensor &t, FlashArgs &p) {
    if (t.src[0] < 0 || t.src[1] < 0 || t.src[2] < 0) return "missing operands";
    const int32_t m = t.src[3];
    if (t.src[4] >= 0) return "attention sinks are not supported";
    const Tensor &tq = g.tensors[t.src[0]], &tk = g.tensors[t.src[1]], &tv = g.tensors[t.src[2]];
    // f16 / f32 rows, or (on the one-query-per-CTA kernel) bf16 and the block types the executor decodes: whole rows
    auto rows_ok = [](const Tensor &x) {
        const TypeTraits *tr = type_traits(x.ty);
        const bool known = x.ty == TLB_TYPE_F16 || x.ty == TLB_TYPE_F32 || x.ty == TLB_TYPE_BF16 || (tr && tr->blck > 1);
        return known && tr && x.nb[0] == (uint64_t)tr->size && x.ne[0] % tr->blck == 0;
    };
    const bool tc_types = (tk.ty == TLB_TYPE_F16 || tk.ty == TLB_TYPE_F32) && (tv.ty == TLB_TYPE_F16 || tv.ty == TLB_TYPE_F32);
    if (tq.ty != TLB_TYPE_F32 || tq.nb[0] != 4 || t.ty != TLB_TYPE_F32) return "queries and result must be f32";
    if (!rows_ok(tk) || !rows_ok(tv)) return "keys and values must be rows of f32, f16, bf16 or a block-quantized type";
    if (!flash_supported(tq.ne[0], tv.ne[0]) || tk.ne[0] != tq.ne[0]) return "head sizes above 512, or keys of another size than the queries";
    if (tk.ne[1] != tv.ne[1] || tk.ne[2] != tv.ne[2] || tk.ne[2] == 0 || tq.ne[2] % tk.ne[2] != 0 || tk.ne[3] != tq.ne[3] || tv.ne[3] != tq.ne[3])
        return "inconsistent shapes";
    if (tc_types && flash_rows_need_alignment(tq.ne[0], tv.ne[0]) &&
        (tk.nb[1] % 16 || tv.nb[1] % 16 || tk.nb[2] % 16 || tv.nb[2] % 16 || tk.nb[3] % 16 || tv.nb[3] % 16 || tq.nb[1] % 8 || tq.nb[2] % 8 || tq.nb[3] % 8))
        return "rows must start on 16-byte boundaries";
    if (t.ne[0] != tv.ne[0] || t.ne[1] != tq.ne[2] || t.ne[2] != tq.ne[1] || t.ne[3] != tq.ne[3] || !t.is_contiguous())
        return "the result must be a contiguous [dv, heads, queries, batch] tensor";
    p = FlashArgs{};
    p.q = view_of(tq);
    p.k = view_of(tk);
    p.v = view_of(tv);
    p.d = (int)tq.ne[0];
    p.dv = (int)tv.ne[0];
    p.nq = (int)tq.ne[1];
    p.nh = (int)tq.ne[2];
    p.nb = (int)tq.ne[3];
    p.nkv = (int)tk.ne[1];
    p.nhkv = (int)tk.ne[2];
    p.k_f32 = tk.ty == TLB_TYPE_F32;
    p.v_f32 = tv.ty == TLB_TYPE_F32;
    p.k_ty = tk.ty;
    p.v_ty = tv.ty;
    p.scale = t.param_f32(0);
    p.max_bias = t.param_f32(1);
    p.softcap = t.param_f32(2);
    if (p.softcap != 0.f) p.scale /= p.softcap;
    p.n_head_log2 = 1;
    while (p.n_head_log2 * 2 <= p.nh) p.n_head_log2 *= 2;
    p.m0 = powf(2.0f, -p.max_bias / (float)p.n_head_log2);
    p.m1 = powf(2.0f, -(p.max_bias / 2.0f) / (float)p.n_head_log2);
    p.m_ne2 = p.m_ne3 = 1;
    if (m >= 0) {
        const Tensor &tm = g.tensors[m];
        if (tm.ty != TLB_TYPE_F16 || tm.nb[0] != 2 || tm.ne[0] < tk.ne[1] || tm.ne[1] < tq.ne[1] || tm.ne[2] < 1 || tm.ne[3] < 1)
            return "the mask must be f16 [keys, >= queries, ...]";
        p.m = view_of(tm);
        p.m_ne2 = (int)tm.ne[2];
        p.m_ne3 = (int)tm.ne[3];
    }
    return nullptr;
}

void lower_flash(L &l) {
    const Tensor &t = l.t();
    FlashArgs p{};
    if (const char *why = flash_args(*l.c.g, t, p)) unsupported(t, why);
    const int32_t q = l.src(0), k = l.src(1), v = l.src(2), m = t.src[3];
    const bool has_mask = m >= 0;
    Place pm;
    if (has_mask) pm = l.place(m);
    const Place pq = l.place(q), pk = l.place(k), pv = l.place(v), pd = l.place(l.id);
    if (flash_tc_supported(p, has_mask)) {
        // prompt-sized: packed operands and mask flags in the node's scratch, tcgen05 kernel
        const int64_t sc = l.c.layout->scratch[l.pos];
        if (sc < 0) throw std::string("attention scratch was not planned");
        Place ps;
        ps.buf = BUF_ARENA;
        ps.off = (uint64_t)sc;
        l.push([=](const RunCtx &r) {
            return launch_flash_attn_tc(p, r.at(pq), r.at(pk), r.at(pv), has_mask ? r.at(pm) : nullptr, (float *)r.at(pd), r.at(ps), r.err, r.stream);
        });
        return;
    }
    // few queries over a long cache: the keys are split over CTAs, partial results in the node's scratch
    flash_split_plan(p, l.c.dev->prop.multiProcessorCount);
    Place ps;
    if (p.parts > 1) {
        const int64_t sc = l.c.layout->scratch[l.pos];
        if (sc < 0) throw std::string("attention scratch was not planned");
        ps.buf = BUF_ARENA;
        ps.off = (uint64_t)sc;
    }
    const bool split = p.parts > 1;
    l.push([=](const RunCtx &r) {
        return launch_flash_attn(p, r.at(pq), r.at(pk), r.at(pv), has_mask ? r.at(pm) : nullptr, (float *)r.at(pd), split ? r.at(ps) : nullptr,
                                 r.stream);
    });
}

// Behind a K-split tensor-core mul_mat (node `mm` right in front of position `pos`) the peer-memory exchange
// reads the partial sums itself (same conditions as in lower_mul_mat, which then leaves them un-added)
void partial_sums_in_front(const LowerCtx &c, int pos, int32_t mm_id, int &n_split, Place &ps) {
    const Graph &g = *c.g;
    n_split = 0;
    if (pos <= 0 || g.nodes[pos - 1] != mm_id || getenv("TLB_SPLITK_REDUCE_LAUNCH")) return;
    const Tensor &mm = g.tensors[mm_id];
    if (mm.op != "MUL_MAT" || mm.src[0] < 0 || mm.src[1] < 0 || mm.src[2] < 0 || !is_qact(g.tensors[mm.src[2]].op) ||
        g.tensors[mm.src[2]].op_params[1] <= 0 || getenv("TLB_MM_GENERIC") || getenv("TLB_NO_TC"))
        return;
    const Tensor &tw = g.tensors[mm.src[0]], &tx = g.tensors[mm.src[1]];
    const bool plain2d = tw.ne[2] * tw.ne[3] * mm.ne[2] * mm.ne[3] == 1 && tw.nb[1] == tw.row_size() && mm.is_contiguous();
    if (!plain2d || tw.ty != TLB_TYPE_Q4_K || !tc_supported(tw.ty, tw.ne[0], tw.ne[1], tx.ne[1])) return;
    const TcPlan tp = tc_plan(tw.ty, tw.ne[0], tw.ne[1], tx.ne[1], c.dev->prop.multiProcessorCount);
    const int64_t sc = c.layout->scratch[pos - 1];
    if (tp.n_split > 1 && tp.n_col_chunks == 1 && sc >= 0) {
        n_split = tp.n_split;
        ps.buf = BUF_ARENA;
        ps.off = (uint64_t)sc;
    }
}

// The ALLREDUCE at position `pos` feeds only the ROW_QUANT right behind it, as the addend of a residual add in
// front of an RMS norm: the two run as one kernel when the peer-memory exchange is in use.
bool exchange_fused_with_row_quant(const LowerCtx &c, int pos) {
    const Graph &g = *c.g;
    if (getenv("TLB_NO_FUSED_EXCHANGE") || pos < 0 || (size_t)pos + 1 >= g.nodes.size()) return false;
    const int32_t ar = g.nodes[pos];
    const Tensor &A = g.tensors[ar], &R = g.tensors[g.nodes[pos + 1]];
    if (A.op != "ALLREDUCE" || R.op != "ROW_QUANT" || R.op_params[0] != ACT_Q8_K || R.op_params[2] != RQ_NORM || R.src[1] != ar || R.src[0] < 0 ||
        R.src[3] < 0)
        return false;
    if (!exchange_row_quant_supported(A.ne[0], A.nrows()) || !A.is_contiguous()) return false;
    const Tensor &X = g.tensors[R.src[0]], &W = g.tensors[R.src[3]];
    if (X.ne[0] != A.ne[0] || X.nrows() != A.nrows() || W.ne[0] != A.ne[0]) return false;
    const int32_t root = g.root(ar);
    for (int32_t k : g.keep)
        if (g.root(k) == root) return false;
    int readers = 0;
    for (size_t i = 0; i < g.nodes.size(); i++) {
        const Tensor &t = g.tensors[g.nodes[i]];
        if ((int)i == pos || t.is_view_op()) continue;
        for (int s = 0; s < 10; s++)
            if (t.src[s] >= 0 && g.root(t.src[s]) == root) readers++;
    }
    return readers == 1;   // the row quantizer
}

// ---- ALLREDUCE (tensor parallelism; no reference counterpart): the node is a view of its source
void lower_allreduce(L &l) {
    const Tensor &t = l.t();
    const int32_t a = l.src(0);
    if (t.ty != TLB_TYPE_F32 || !t.is_contiguous()) unsupported(t, "allreduce takes a contiguous f32 tensor");
    if (l.c.g->root(l.id) != l.c.g->root(a)) unsupported(t, "allreduce works in place on its source");
    const Place pd = l.place(l.id);
    const size_t n = (size_t)t.nelements();
    tlb_device *dev = l.c.dev;
    int n_split = 0;
    Place ps;
    partial_sums_in_front(l.c, l.pos, a, n_split, ps);
    // the exchange may be done by the row quantizer that follows (fused kernel): then this node launches nothing
    const bool fused_next = exchange_fused_with_row_quant(l.c, l.pos);
    l.push([=](const RunCtx &r) {
        if (fused_next && comm_p2p_takes(dev, n)) return cudaSuccess;
        if (n_split > 0 && comm_p2p_takes(dev, n))
            return comm_allreduce_f32(dev, (float *)r.at(pd), n, r.stream, r.err, (const float *)r.at(ps), n_split);
        return comm_allreduce_f32(dev, (float *)r.at(pd), n, r.stream, r.err);
    });
}

}  // namespace

uint64_t node_scratch_bytes(const Graph &g, int32_t id, int sm_count) {
    const Tensor &t = g.tensors[id];
    if (t.op == "CUSTOM") {
        PagedGeom pg{};
        if (paged_geom(g, t, sm_count, pg)) return paged_scratch_bytes(pg);
    }
    if (t.op == "FLASH_ATTN_EXT") {
        FlashArgs p{};
        if (flash_args(g, t, p) == nullptr) {
            if (flash_tc_supported(p, t.src[3] >= 0)) return flash_tc_scratch_bytes(p, t.src[3] >= 0);
            flash_split_plan(p, sm_count);
            return flash_split_scratch_bytes(p);
        }
    }
    if (t.op == "MUL_MAT_GROUP") {
        const Tensor &tx = g.tensors[t.src[1]];
        int64_t Msum = 0;
        for (int s : {0, 3, 5})
            if (t.src[s] >= 0) Msum += g.tensors[t.src[s]].ne[1];
        return mmq_tc_plan(tx.ne[0], Msum, tx.ne[1], sm_count).partial_bytes;
    }
    if (t.op == "MUL_MAT" && t.src[0] >= 0 && t.src[1] >= 0 && t.src[2] >= 0 && is_qact(g.tensors[t.src[2]].op) &&
        g.tensors[t.src[2]].op_params[1] > 0) {
        // split-K partial sums of the tensor-core path
        const Tensor &tw = g.tensors[t.src[0]], &tx = g.tensors[t.src[1]];
        if (tw.ne[2] * tw.ne[3] * t.ne[2] * t.ne[3] == 1 && tc_supported(tw.ty, tw.ne[0], tw.ne[1], tx.ne[1]))
            return tc_plan(tw.ty, tw.ne[0], tw.ne[1], tx.ne[1], sm_count).partial_bytes;
    }
    return 0;
}

// ---- image ops (lower.rs:366-382 im2col, 392-420 upscale, 469-482 pool_2d, 506-539 conv_2d_dw / pad)
void lower_image(L &l) {
    const Tensor &t = l.t();
    const std::string &op = t.op;
    auto float_type = [](uint32_t ty) { return ty == TLB_TYPE_F32 || ty == TLB_TYPE_F16 || ty == TLB_TYPE_BF16; };
    const Place pd = l.place(l.id);
    if (op == "IM2COL") {
        const int32_t k = l.src(0), x = l.src(1);
        const Tensor &tk = l.T(k), &tx = l.T(x);
        if (!float_type(tx.ty) || !float_type(t.ty)) unsupported(t, "im2col takes f32 / f16 / bf16 data");
        Im2colArgs p{};
        p.x = view_of(tx);
        p.d = view_of(t);
        p.xty = tx.ty;
        p.dty = t.ty;
        p.s0 = t.op_params[0]; p.s1 = t.op_params[1]; p.p0 = t.op_params[2]; p.p1 = t.op_params[3]; p.d0 = t.op_params[4]; p.d1 = t.op_params[5];
        p.is2d = t.op_params[6] == 1;
        p.KW = tk.ne[0];
        p.KH = p.is2d ? tk.ne[1] : 1;
        p.IH = p.is2d ? tx.ne[1] : 1;
        p.IW = tx.ne[0];
        if (p.s0 < 1 || (p.is2d && p.s1 < 1) || p.KW < 1 || p.KH < 1 || t.ne[0] % (p.KW * p.KH) != 0) unsupported(t, "inconsistent im2col parameters");
        const Place px = l.place(x);
        l.push([=](const RunCtx &r) { return launch_im2col(p, r.at(px), r.at(pd), r.stream); });
    } else if (op == "UPSCALE") {
        const int32_t a = l.src(0);
        const Tensor &ta = l.T(a);
        if (ta.ty != TLB_TYPE_F32 || t.ty != TLB_TYPE_F32) unsupported(t, "upscale takes f32");
        const int32_t flags = t.op_params[0];
        UpscaleArgs p{};
        p.a = view_of(ta);
        p.d = view_of(t);
        p.mode = flags & 0xFF;
        p.antialias = (flags & (1 << 9)) != 0;
        if (p.mode < 0 || p.mode > 2) unsupported(t, "unknown upscale mode");
        if (p.antialias && p.mode != 1) unsupported(t, "antialiasing is bilinear only");
        for (int i = 0; i < 4; i++)
            if (ta.ne[i] < 1) unsupported(t, "empty source");
        float sf[4];
        for (int i = 0; i < 4; i++) sf[i] = (float)t.ne[i] / (float)ta.ne[i];
        p.poff = 0.5f;
        if (flags & (1 << 8)) {   // align corners
            p.poff = 0.0f;
            for (int i = 0; i < 2; i++)
                if (t.ne[i] > 1 && ta.ne[i] > 1) sf[i] = (float)(t.ne[i] - 1) / (float)(ta.ne[i] - 1);
        }
        p.sf0 = sf[0]; p.sf1 = sf[1]; p.sf2 = sf[2]; p.sf3 = sf[3];
        const Place pa = l.place(a);
        l.push([=](const RunCtx &r) { return launch_upscale(p, r.at(pa), r.at(pd), r.stream); });
    } else if (op == "POOL_2D") {
        const int32_t a = l.src(0);
        const Tensor &ta = l.T(a);
        if (!float_type(ta.ty) || !float_type(t.ty)) unsupported(t, "pooling takes f32 / f16 / bf16");
        Pool2dArgs p{};
        p.a = view_of(ta);
        p.d = view_of(t);
        p.aty = ta.ty;
        p.dty = t.ty;
        p.kind = t.op_params[0]; p.k0 = t.op_params[1]; p.k1 = t.op_params[2]; p.s0 = t.op_params[3]; p.s1 = t.op_params[4];
        p.p0 = t.op_params[5]; p.p1 = t.op_params[6];
        if (p.kind != 0 && p.kind != 1) unsupported(t, "unknown pooling op");
        if (p.k0 < 1 || p.k1 < 1 || p.s0 < 1 || p.s1 < 1 || t.ne[2] != ta.ne[2] || t.ne[3] != ta.ne[3]) unsupported(t, "inconsistent pooling parameters");
        const Place pa = l.place(a);
        l.push([=](const RunCtx &r) { return launch_pool_2d(p, r.at(pa), r.at(pd), r.stream); });
    } else if (op == "CONV_2D_DW") {
        const int32_t k = l.src(0), x = l.src(1);
        const Tensor &tk = l.T(k), &tx = l.T(x);
        if (!float_type(tk.ty) || !float_type(tx.ty) || !float_type(t.ty)) unsupported(t, "depthwise convolution takes f32 / f16 / bf16");
        if (tk.ne[2] != 1 || tk.ne[3] != tx.ne[2] || t.ne[2] != tx.ne[2] || t.ne[3] != tx.ne[3]) unsupported(t, "inconsistent shapes");
        ConvDwArgs p{};
        p.k = view_of(tk);
        p.x = view_of(tx);
        p.d = view_of(t);
        p.kty = tk.ty; p.xty = tx.ty; p.dty = t.ty;
        p.s0 = t.op_params[0]; p.s1 = t.op_params[1]; p.p0 = t.op_params[2]; p.p1 = t.op_params[3]; p.d0 = t.op_params[4]; p.d1 = t.op_params[5];
        if (p.s0 < 1 || p.s1 < 1) unsupported(t, "strides must be positive");
        const Place pk = l.place(k), px = l.place(x);
        l.push([=](const RunCtx &r) { return launch_conv_2d_dw(p, r.at(pk), r.at(px), r.at(pd), r.stream); });
    } else {
        const int32_t a = l.src(0);
        const Tensor &ta = l.T(a);
        if (ta.ty != t.ty) unsupported(t, "padding keeps the element type");
        const uint64_t es = type_traits(t.ty)->size;
        if (type_traits(t.ty)->blck != 1 || (es != 2 && es != 4)) unsupported(t, "padding takes 2- or 4-byte elements");
        PadArgs p{};
        p.a = view_of(ta);
        p.d = view_of(t);
        p.elem_bytes = (int)es;
        if (op == "PAD") {
            if (t.op_params[8] != 0) unsupported(t, "circular padding");
            for (int i = 0; i < 4; i++) {
                p.lp[i] = t.op_params[2 * i];
                if (p.lp[i] < 0 || t.op_params[2 * i + 1] < 0 || t.ne[i] != ta.ne[i] + p.lp[i] + t.op_params[2 * i + 1]) unsupported(t, "inconsistent padding");
            }
        } else {
            p.reflect = 1;
            p.lp[0] = t.op_params[0];
            if (p.lp[0] < 0 || t.op_params[1] < 0 || p.lp[0] >= ta.ne[0] || t.op_params[1] >= ta.ne[0] || t.ne[0] != ta.ne[0] + p.lp[0] + t.op_params[1] ||
                t.ne[1] != ta.ne[1] || t.ne[2] != ta.ne[2] || t.ne[3] != ta.ne[3])
                unsupported(t, "reflection needs pads shorter than the row");
        }
        const Place pa = l.place(a);
        l.push([=](const RunCtx &r) { return launch_pad(p, r.at(pa), r.at(pd), r.stream); });
    }
}

void lower_node(const LowerCtx &c, int32_t id, int pos, std::vector<Dispatch> &out) {
    const Tensor &t = c.g->tensors[id];
    if (t.is_view_op() || t.nelements() == 0) return;
    L l{c, id, pos, out};
    const std::string &op = t.op;
    if (op == "QUANT_ACT") return lower_quant_act(l);
    if (op == "ROW_QUANT") return lower_row_quant(l);
    for (int s : t.src)
        if (s >= 0) {
            const uint32_t ty = c.g->tensors[s].ty;
            if (!(plain(ty) || gemv_type(ty) || decoded_type(ty)) && !is_qact(c.g->tensors[s].op)) unsupported(t, "operand type");
        }
    if (!plain(t.ty)) unsupported(t, "operand type");
    if (op == "ADD" || op == "SUB" || op == "MUL" || op == "DIV") return lower_bin(l);
    if (op == "SCALE" || op == "FILL" || op == "CLAMP" || op == "LEAKY_RELU" || op == "SQR" || op == "SQRT" || op == "SIN" ||
        op == "COS" || op == "LOG" || op == "UNARY")
        return lower_unary(l);
    if (op == "GLU") return lower_glu(l);
    if (op == "NORM" || op == "RMS_NORM") return lower_norm(l, false);
    if (op == "RMS_NORM_MUL") return lower_norm(l, true);
    if (op == "ROPE") return lower_rope(l);
    if (op == "ROPE_KV_WRITE") return lower_rope_kv(l);
    if (op == "SOFT_MAX") return lower_soft_max(l);
    if (op == "GET_ROWS") return lower_get_rows(l);
    if (op == "SET_ROWS") return lower_set_rows(l);
    if (op == "DUP" || op == "CPY" || op == "CONT") return lower_cpy(l);
    if (op == "ARGMAX") return lower_argmax(l);
    if (op == "CONCAT" || op == "REPEAT" || op == "SUM_ROWS" || op == "MEAN" || op == "ARANGE") return lower_simple(l);
    if (op == "IM2COL" || op == "UPSCALE" || op == "POOL_2D" || op == "CONV_2D_DW" || op == "PAD" || op == "PAD_REFLECT_1D") return lower_image(l);
    if (op == "MUL_MAT") return lower_mul_mat(l);
    if (op == "MUL_MAT_GROUP") return lower_mul_mat_group(l);
    if (op == "CUSTOM") return lower_custom(l);
    if (op == "FLASH_ATTN_EXT") return lower_flash(l);
    if (op == "ALLREDUCE") return lower_allreduce(l);
    unsupported(t, "op not implemented in the native CUDA backend");
}

// ---------------------------------------------------------------------------- IR rewrites
void fuse_row_producers(Graph &g);
void fuse_rope_cache(Graph &g);
void fuse_mul_mat_groups(Graph &g);
void fuse_attn_quant(Graph &g);
// Readers of every root (views of a tensor count for the root), as fuse.rs:56-63 requires.
void rewrite_graph(Graph &g) {
    const size_t nt0 = g.tensors.size();
    auto readers_of = [&](std::vector<int> &readers) {
        readers.assign(g.tensors.size(), 0);
        for (int32_t n : g.nodes) {
            const Tensor &t = g.tensors[n];
            for (int s : t.src)
                if (s >= 0) readers[g.root(s)]++;
        }
        for (int32_t k : g.keep) readers[g.root(k)] += 2;  // kept tensors never fuse away
    };
    std::vector<int> readers;
    readers_of(readers);
    std::vector<int> pos_of(nt0, -1);
    for (size_t i = 0; i < g.nodes.size(); i++) pos_of[g.nodes[i]] = (int)i;
    std::vector<char> dead(g.nodes.size(), 0);
    const char *nf = getenv("TL_NATIVE_NOFUSE");
    const std::string nofuse = nf ? nf : "";
    // "1" turns every fusion off, a list of names only those
    auto enabled = [&](const char *name) { return nofuse != "1" && nofuse.find(name) == std::string::npos; };

    for (size_t i = 0; i < g.nodes.size(); i++) {
        const int32_t id = g.nodes[i];
        Tensor &t = g.tensors[id];
        if (t.op != "MUL" || t.view_src >= 0) continue;
        // RMS_NORM + MUL -> RMS_NORM_MUL (fuse.rs:88-113)
        for (int side = 0; side < 2 && enabled("RMS_NORM_MUL"); side++) {
            const int32_t a = t.src[side], w = t.src[1 - side];
            if (a < 0 || w < 0) continue;
            Tensor &n = g.tensors[a];
            if (n.op != "RMS_NORM" || n.view_src >= 0 || readers[a] != 1 || pos_of[a] < 0 || dead[pos_of[a]]) continue;
            const Tensor &tw = g.tensors[w];
            if (t.ty != 0 || n.ty != 0 || tw.ty != 0 || !t.is_contiguous() || tw.nb[0] != 4) continue;
            bool same = true;
            for (int k = 0; k < 4; k++) same = same && t.ne[k] == n.ne[k];
            if (!same || tw.ne[0] == 0 || n.ne[0] % tw.ne[0] != 0) continue;
            bool bc = true;
            for (int k = 1; k < 4; k++) bc = bc && tw.ne[k] != 0 && t.ne[k] % tw.ne[k] == 0;
            if (!bc || n.src[0] < 0 || g.tensors[n.src[0]].nb[0] != 4) continue;
            t.op = "RMS_NORM_MUL";
            t.op_params[15] = n.op_params[0];  // eps moves to slot 15
            t.src[0] = n.src[0];
            t.src[1] = w;
            dead[pos_of[a]] = 1;
            break;
        }
        if (t.op != "MUL") continue;
        // act(g) * u -> GLU (the gated MLP of stdlib/nn.ss; FUSED_GU of fuse_tree.rs without the matmuls)
        for (int side = 0; side < 2 && enabled("GLU"); side++) {
            const int32_t a = t.src[side], u = t.src[1 - side];
            if (a < 0 || u < 0) continue;
            const Tensor &n = g.tensors[a];
            if (n.op != "UNARY" || n.view_src >= 0 || readers[a] != 1 || pos_of[a] < 0 || dead[pos_of[a]]) continue;
            int glu = -1;
            switch (n.op_params[0]) {
                case 6: glu = 0; break;   // RELU  -> REGLU
                case 8: glu = 1; break;   // GELU  -> GEGLU
                case 10: glu = 2; break;  // SILU  -> SWIGLU
                case 16: glu = 4; break;  // GELU_ERF
                case 9: glu = 5; break;   // GELU_QUICK
            }
            const int32_t gsrc = n.src[0];
            if (glu < 0 || gsrc < 0) continue;
            const Tensor &tg = g.tensors[gsrc], &tu = g.tensors[u];
            if (t.ty != 0 || tg.ty != 0 || tu.ty != 0 || !t.is_contiguous() || !tg.is_contiguous() || !tu.is_contiguous()) continue;
            bool same = true;
            for (int k = 0; k < 4; k++) same = same && t.ne[k] == tg.ne[k] && t.ne[k] == tu.ne[k];
            if (!same) continue;
            t.op = "GLU";
            for (int k = 0; k < 16; k++) t.op_params[k] = 0;
            t.op_params[0] = glu;
            t.src[0] = gsrc;
            t.src[1] = u;
            dead[pos_of[a]] = 1;
            break;
        }
    }

    // Quantize each distinct activation once: a QUANT_ACT node in front of the first quantized
    // MUL_MAT that reads it, shared by later ones until something writes its storage again.
    std::vector<int32_t> nodes;
    std::map<std::pair<int32_t, int>, int32_t> cache;  // (activation tensor, kind) -> QUANT_ACT tensor
    for (size_t i = 0; i < g.nodes.size(); i++) {
        if (dead[i]) continue;
        const int32_t id = g.nodes[i];
        {
            // a node that writes into storage an activation lives in invalidates its quantized copy
            const int32_t root = g.root(id);
            for (auto it = cache.begin(); it != cache.end();) {
                if (g.root(it->first.first) == root && !g.tensors[id].is_view_op()) it = cache.erase(it);
                else ++it;
            }
        }
        Tensor &t = g.tensors[id];
        if (t.op == "MUL_MAT" && t.src[0] >= 0 && t.src[1] >= 0 && gemv_type(g.tensors[t.src[0]].ty)) {
            const Tensor tw = g.tensors[t.src[0]];   // by value: the tensor vector grows below
            const int32_t x = t.src[1];
            const Tensor tx = g.tensors[x];
            const int kind = act_kind_for(tw.ty);
            const int64_t blk = kind == ACT_Q8_K ? 256 : 32;
            bool ok = tx.ty == 0 && tx.nb[0] == 4 && tx.ne[0] % blk == 0 && tx.nelements() > 0 && tx.nb[1] % 16 == 0;
            // columns must be uniformly strided
            if (ok && tx.ne[2] > 1) ok = tx.nb[2] == tx.nb[1] * (uint64_t)tx.ne[1];
            if (ok && tx.ne[3] > 1) ok = tx.nb[3] == tx.nb[1] * (uint64_t)tx.ne[1] * (uint64_t)tx.ne[2];
            if (ok) {
                auto key = std::make_pair(x, kind);
                auto it = cache.find(key);
                int32_t qa;
                if (it != cache.end()) {
                    qa = it->second;
                } else {
                    Tensor q;
                    q.ty = TLB_TYPE_I8;
                    q.op = "QUANT_ACT";
                    q.op_params[0] = kind;
                    q.src[0] = x;
                    q.opaque_bytes = act_layout(kind, tx.ne[0], tx.nrows()).bytes;
                    q.ne[0] = (int64_t)q.opaque_bytes;
                    q.nb[0] = 1;
                    q.nb[1] = q.nb[2] = q.nb[3] = q.opaque_bytes;
                    q.name = tx.name + ".q8";
                    qa = (int32_t)g.tensors.size();
                    g.tensors.push_back(q);
                    nodes.push_back(qa);
                    cache[key] = qa;
                }
                g.tensors[id].src[2] = qa;
                // a consumer that takes the tensor-core path also needs the packed blobs behind the Q8_K block
                const Tensor &mm = g.tensors[id];
                const bool plain2d = tw.ne[2] * tw.ne[3] * mm.ne[2] * mm.ne[3] == 1 && tw.nb[1] == tw.row_size();
                if (plain2d && tc_supported(tw.ty, tx.ne[0], tw.ne[1], tx.ne[1]) && !getenv("TLB_NO_TC")) {
                    const TcPlan tp = tc_plan(tw.ty, tx.ne[0], tw.ne[1], tx.ne[1], 148);
                    Tensor &q = g.tensors[qa];
                    q.op_params[1] = tp.npad;
                    q.opaque_bytes = act_layout(kind, tx.ne[0], tx.nrows()).bytes + tp.blob_bytes;
                    q.ne[0] = (int64_t)q.opaque_bytes;
                    q.nb[1] = q.nb[2] = q.nb[3] = q.opaque_bytes;
                }
            }
        }
        nodes.push_back(id);
    }
    g.nodes.swap(nodes);
    if (enabled("ROW_QUANT")) fuse_row_producers(g);
    if (enabled("ROW_QUANT") && enabled("ATTN_QUANT")) fuse_attn_quant(g);
    if (enabled("ROPE_KV_WRITE")) fuse_rope_cache(g);
    if (enabled("MUL_MAT_GROUP")) fuse_mul_mat_groups(g);
}

// The f16 output of paged attention, cast and quantized for the output projection (a ROW_QUANT node in RQ_F16 mode right
// behind the attention): the attention kernel quantizes its rows itself when it runs without a context split (one
// launch less per layer). The ROW_QUANT node leaves the node list; its tensor becomes src[9] of the attention node, which
// also makes the planner keep it alive from that position on.
void fuse_attn_quant(Graph &g) {
    const size_t nn = g.nodes.size();
    std::vector<int> pos_of(g.tensors.size(), -1);
    for (size_t i = 0; i < nn; i++) pos_of[g.nodes[i]] = (int)i;
    std::vector<char> dead(nn, 0);
    for (size_t qi = 0; qi < nn; qi++) {
        const int32_t qid = g.nodes[qi];
        const Tensor &Q = g.tensors[qid];
        if (Q.op != "ROW_QUANT" || Q.op_params[2] != RQ_F16 || Q.op_params[0] != ACT_Q8_K || Q.src[0] < 0 || Q.src[5] < 0) continue;
        const int32_t src = Q.src[0], root = g.root(src);
        const int ap = pos_of[root];
        if (ap < 0 || ap >= (int)qi) continue;
        Tensor &A = g.tensors[root];
        if (A.op != "CUSTOM" || paged_ud(A).kind != 1 || A.src[9] >= 0) continue;
        bool only_views = true;
        for (int i = ap + 1; i < (int)qi; i++) only_views = only_views && g.tensors[g.nodes[i]].is_view_op();
        if (!only_views) continue;
        // the quantizer reads the whole output as rows of heads * head size, one per sequence
        const Tensor &S = g.tensors[src], &shape = g.tensors[Q.src[5]];
        if (S.ty != TLB_TYPE_F16 || !S.is_contiguous() || S.view_offs != 0 || S.nelements() != A.nelements()) continue;
        if (shape.ne[0] != A.ne[0] * A.ne[1] || shape.nrows() != A.ne[2]) continue;
        PagedGeom pg{};
        if (!paged_geom(g, A, 148, pg) || pg.n_chunks != 1 || !paged_quant_fusable(pg)) continue;
        A.src[9] = qid;
        dead[qi] = 1;
    }
    std::vector<int32_t> out;
    for (size_t i = 0; i < nn; i++)
        if (!dead[i]) out.push_back(g.nodes[i]);
    g.nodes.swap(out);
}

// Fold the producer of a quantized activation into its QUANT_ACT node (k_fused.cu): RMS_NORM_MUL
// (optionally with the residual ADD in front of it), GLU(swiglu) and the f16 -> f32 cast of the
// attention output. Legality follows vulkan/fuse.rs:56-63: the folded intermediates have no other
// reader, are not kept, and nothing between the folded nodes and the fused one touches them.
void fuse_row_producers(Graph &g) {
    const size_t nn = g.nodes.size();
    std::vector<int> pos_of(g.tensors.size(), -1);
    for (size_t i = 0; i < nn; i++) pos_of[g.nodes[i]] = (int)i;
    std::vector<char> kept(g.tensors.size(), 0);
    for (int32_t k : g.keep) kept[g.root(k)] = 1;
    // a MUL_MAT that carries a QUANT_ACT of its activation never reads the f32 activation itself
    auto really_reads = [&](const Tensor &t, int slot) {
        return !(t.op == "MUL_MAT" && slot == 1 && t.src[2] >= 0 && is_qact(g.tensors[t.src[2]].op) &&
                 gemv_type(g.tensors[t.src[0]].ty));
    };
    // readers of a root among the nodes, by position
    auto readers = [&](int32_t root, std::vector<int> &out) {
        out.clear();
        for (size_t i = 0; i < nn; i++) {
            const Tensor &t = g.tensors[g.nodes[i]];
            for (int s = 0; s < 10; s++)
                if (t.src[s] >= 0 && g.root(t.src[s]) == root && really_reads(t, s)) out.push_back((int)i);
        }
    };
    auto dense_rows = [&](const Tensor &t, int64_t es) {
        if (t.nb[0] != (uint64_t)es) return false;
        if (t.ne[2] > 1 && t.nb[2] != t.nb[1] * (uint64_t)t.ne[1]) return false;
        if (t.ne[3] > 1 && t.nb[3] != t.nb[1] * (uint64_t)t.ne[1] * (uint64_t)t.ne[2]) return false;
        return t.nb[1] % 16 == 0;
    };
    std::vector<char> dead(nn, 0);
    std::vector<int> rd;
    for (size_t qi = 0; qi < nn; qi++) {
        const int32_t qid = g.nodes[qi];
        if (g.tensors[qid].op != "QUANT_ACT") continue;
        // Q8_K activations (Q4_K weights), or the Q8_0 activations of the prompt mul_mat (operand blobs of 256 columns)
        const bool q80 = g.tensors[qid].op_params[0] == ACT_Q8_0;
        if (q80 && g.tensors[qid].op_params[1] != 256) continue;
        const int32_t x = g.tensors[qid].src[0];
        const Tensor X = g.tensors[x];
        if (X.ty != 0 || !row_quant_supported(X.ne[0]) || !dense_rows(X, 4)) continue;
        const int32_t xroot = g.root(x);
        if (kept[xroot]) continue;
        const int xp = pos_of[xroot];
        if (xp < 0 || dead[xp]) continue;
        const Tensor P = g.tensors[xroot];   // producer of the storage X views
        // every reader of the producer's storage must be this QUANT_ACT (views of it launch nothing)
        readers(xroot, rd);
        bool only_q = true;
        // (a cast lists itself as src[1], ggml.c:3549-3563, so the producer shows up as its own reader)
        for (int r : rd) only_q = only_q && (r == (int)qi || r == xp || g.tensors[g.nodes[r]].is_view_op());
        if (!only_q) continue;
        Tensor &Q = g.tensors[qid];
        if (P.op == "RMS_NORM_MUL" && xroot == x) {
            const int32_t a = P.src[0], w = P.src[1];
            const Tensor &A = g.tensors[a], &W = g.tensors[w];
            if (A.ty != 0 || W.ty != 0 || W.nb[0] != 4 || W.ne[1] * W.ne[2] * W.ne[3] != 1 || !dense_rows(A, 4)) continue;
            if (q80 && !row_quant_q80_supported(X.ne[0], RQ_NORM)) continue;
            Q.op = "ROW_QUANT";
            Q.op_params[2] = RQ_NORM;
            Q.op_params[15] = P.op_params[15];
            Q.src[0] = a;
            Q.src[1] = -1;
            Q.src[3] = w;
            dead[xp] = 1;
            // residual ADD in front of the norm: computed (and written back) by the same launch
            const int32_t aroot = g.root(a);
            const int ap = pos_of[aroot];
            if (a == aroot && ap >= 0 && !dead[ap] && g.tensors[a].op == "ADD") {
                const Tensor R = g.tensors[a];
                const int32_t s0 = R.src[0], s1 = R.src[1];
                bool ok = s0 >= 0 && s1 >= 0 && g.tensors[s0].ty == 0 && g.tensors[s1].ty == 0 && R.is_contiguous() &&
                          dense_rows(g.tensors[s0], 4) && dense_rows(g.tensors[s1], 4);
                for (int k = 0; ok && k < 4; k++) ok = g.tensors[s0].ne[k] == R.ne[k] && g.tensors[s1].ne[k] == R.ne[k];
                // nobody may read the sum between the ADD's old position and the fused node
                readers(aroot, rd);
                for (int r : rd) ok = ok && (r >= (int)qi || r == xp);
                if (ok) {
                    Q.src[0] = s0;
                    Q.src[1] = s1;
                    Q.src[4] = a;   // the sum is written into the ADD's own tensor
                    dead[ap] = 1;
                }
            }
        } else if (P.op == "GLU" && xroot == x && P.op_params[0] == 2 && P.src[0] >= 0 && P.src[1] >= 0) {
            const Tensor &G0 = g.tensors[P.src[0]], &U0 = g.tensors[P.src[1]];
            if (G0.ty != 0 || U0.ty != 0 || !dense_rows(G0, 4) || !dense_rows(U0, 4)) continue;
            Q.op = "ROW_QUANT";
            Q.op_params[2] = RQ_GLU;
            Q.src[0] = P.src[0];
            Q.src[1] = P.src[1];
            dead[xp] = 1;
        } else if (P.op == "CPY" && P.src[0] >= 0 && g.tensors[P.src[0]].ty == TLB_TYPE_F16 && P.is_contiguous() &&
                   g.tensors[P.src[0]].is_contiguous() && P.view_src < 0) {
            Q.op = "ROW_QUANT";
            Q.op_params[2] = RQ_F16;
            Q.src[0] = P.src[0];
            Q.src[1] = -1;
            Q.src[5] = x;   // keeps the shape of the activation matrix (a view of the folded cast)
            dead[xp] = 1;
        }
    }
    std::vector<int32_t> out;
    for (size_t i = 0; i < nn; i++)
        if (!dead[i]) out.push_back(g.nodes[i]);
    g.nodes.swap(out);
}


// rope(q) -> cast, rope(k) -> cast, v -> cast, cache write: one ROPE_KV_WRITE node in place of the
// cache write (decode-step shape of scheme/core.ss:222-271 callers). Legality as for the other
// fusions: every folded intermediate has exactly one reader, is not kept, and is a plain f32/f16
// tensor of the expected shape; both ropes share position tensor and parameters.
void fuse_rope_cache(Graph &g) {
    const size_t nn = g.nodes.size();
    std::vector<int> pos_of(g.tensors.size(), -1);
    for (size_t i = 0; i < nn; i++) pos_of[g.nodes[i]] = (int)i;
    std::vector<char> kept(g.tensors.size(), 0);
    for (int32_t k : g.keep) kept[g.root(k)] = 1;
    // readers of a root by node position; a cast lists itself as src[1] and is not its own reader
    auto n_readers = [&](int32_t root, int self_pos) {
        int n = 0;
        for (size_t i = 0; i < nn; i++) {
            if ((int)i == self_pos) continue;
            const Tensor &t = g.tensors[g.nodes[i]];
            if (t.is_view_op()) continue;
            for (int s = 0; s < 10; s++)
                if (t.src[s] >= 0 && g.root(t.src[s]) == root) { n++; break; }
        }
        return n;
    };
    // a cast to f16 of (a view of) `want_op`'s result, read once: returns the producing node or -1
    auto cast_of = [&](int32_t c16, const char *want_op) -> int32_t {
        if (c16 < 0 || g.root(c16) != c16) return -1;
        const Tensor &C = g.tensors[c16];
        if (C.op != "CPY" || C.ty != TLB_TYPE_F16 || !C.is_contiguous() || C.src[0] < 0 || kept[c16] || pos_of[c16] < 0) return -1;
        const int32_t src = g.root(C.src[0]);
        const Tensor &S = g.tensors[src];
        if (S.ty != TLB_TYPE_F32 || kept[src]) return -1;
        if (want_op && (S.op != want_op || pos_of[src] < 0)) return -1;
        if (!g.tensors[C.src[0]].is_contiguous()) return -1;
        return src;
    };
    std::vector<char> dead(nn, 0);
    for (size_t ci = 0; ci < nn; ci++) {
        const int32_t cid = g.nodes[ci];
        Tensor &Cw = g.tensors[cid];
        if (Cw.op != "CUSTOM" || paged_ud(Cw).kind != 2) continue;
        const PagedUd u = paged_ud(Cw);
        const int32_t k16 = Cw.src[0], v16 = Cw.src[1];
        const int32_t rk = cast_of(k16, "ROPE");
        const int32_t vsrc = cast_of(v16, nullptr);
        if (rk < 0 || vsrc < 0) continue;
        // the attention node that reads the same pools, and its query
        int ai = -1;
        for (size_t i = ci + 1; i < nn && ai < 0; i++) {
            const Tensor &A = g.tensors[g.nodes[i]];
            if (A.op == "CUSTOM" && paged_ud(A).kind == 1 && A.src[1] == Cw.src[2] && A.src[2] == Cw.src[3]) ai = (int)i;
        }
        if (ai < 0) continue;
        const int32_t q16 = g.tensors[g.nodes[ai]].src[0];
        const int32_t rq = cast_of(q16, "ROPE");
        if (rq < 0) continue;
        const Tensor RQ = g.tensors[rq], RK = g.tensors[rk];
        bool ok = RQ.src[1] == RK.src[1] && RQ.src[2] == RK.src[2] && RQ.src[0] >= 0 && RK.src[0] >= 0;
        for (int i = 0; ok && i < 16; i++) ok = RQ.op_params[i] == RK.op_params[i];
        if (!ok) continue;
        const Tensor &QI = g.tensors[RQ.src[0]], &KI = g.tensors[RK.src[0]], &VI = g.tensors[g.tensors[v16].src[0]];
        const int64_t hs = QI.ne[0], tokens = QI.ne[2];
        ok = QI.ty == 0 && KI.ty == 0 && VI.ty == 0 && QI.nb[0] == 4 && KI.nb[0] == 4 && VI.nb[0] == 4 && QI.ne[3] == 1 && KI.ne[3] == 1 &&
             KI.ne[0] == hs && KI.ne[1] == u.kv_heads && KI.ne[2] == tokens && VI.ne[0] == hs * u.kv_heads && VI.nrows() == tokens &&
             hs % 2 == 0 && hs <= 2048 && QI.nb[1] % 8 == 0 && VI.nb[1] % 8 == 0 && g.tensors[RQ.src[1]].ty == TLB_TYPE_I32 &&
             g.tensors[RQ.src[1]].ne[0] == tokens && g.tensors[q16].ne[0] == hs && g.tensors[k16].nelements() == hs * u.kv_heads * tokens &&
             (RQ.src[2] < 0 || (g.tensors[RQ.src[2]].ty == 0 && g.tensors[RQ.src[2]].nb[0] == 4));
        // one reader each: rope results by their casts, casts by the cache write / the attention
        ok = ok && n_readers(rq, pos_of[rq]) == 1 && n_readers(rk, pos_of[rk]) == 1 && n_readers(k16, pos_of[k16]) == 1 &&
             n_readers(v16, pos_of[v16]) == 1 && n_readers(q16, pos_of[q16]) == 1;
        // the folded nodes all sit before the attention; the fused node takes the cache write's place
        ok = ok && pos_of[rq] < (int)ci && pos_of[rk] < (int)ci && pos_of[k16] < (int)ci && pos_of[v16] < (int)ci && pos_of[q16] < ai;
        if (!ok) continue;
        const int32_t pools[2] = {Cw.src[2], Cw.src[3]};
        const int32_t slots = Cw.src[4];
        Cw.op = "ROPE_KV_WRITE";
        for (int i = 0; i < 16; i++) Cw.op_params[i] = RQ.op_params[i];
        Cw.op_params[12] = u.kv_heads;
        Cw.op_params[13] = u.block_size;
        for (int i = 0; i < 10; i++) Cw.src[i] = -1;
        Cw.src[0] = RQ.src[0];
        Cw.src[1] = RK.src[0];
        Cw.src[2] = g.tensors[v16].src[0];
        Cw.src[3] = RQ.src[1];
        Cw.src[4] = RQ.src[2];
        Cw.src[5] = pools[0];
        Cw.src[6] = pools[1];
        Cw.src[7] = slots;
        Cw.src[8] = q16;   // written by this node
        dead[pos_of[rq]] = dead[pos_of[rk]] = dead[pos_of[k16]] = dead[pos_of[v16]] = dead[pos_of[q16]] = 1;
    }
    std::vector<int32_t> out;
    for (size_t i = 0; i < nn; i++)
        if (!dead[i]) out.push_back(g.nodes[i]);
    g.nodes.swap(out);
}


// Consecutive tensor-core mul_mats over the same quantized activations (wq, wk, wv of a layer; gate and up)
// become one MUL_MAT_GROUP launch: each of wq / wk / wv alone leaves most SMs idle (32 / 8 / 8 row tiles on
// 148 SMs), and gate + up (2 x 112 tiles) together are enough work for the stream-K schedule, which gives
// every SM the same number of super-blocks instead of one wave of 112 tiles twice. Nothing reads a member's result before the
// last member, because the members are adjacent in node order.
void fuse_mul_mat_groups(Graph &g) {
    const size_t nn = g.nodes.size();
    std::vector<char> dead(nn, 0);
    auto eligible = [&](const Tensor &t) {
        if (t.op != "MUL_MAT" || t.src[0] < 0 || t.src[1] < 0 || t.src[2] < 0) return false;
        const Tensor &tw = g.tensors[t.src[0]], &tx = g.tensors[t.src[1]], &q = g.tensors[t.src[2]];
        if (!is_qact(q.op) || q.op_params[1] <= 0 || tw.ty != TLB_TYPE_Q4_K) return false;
        if (tw.ne[2] * tw.ne[3] * t.ne[2] * t.ne[3] != 1 || tw.nb[1] != tw.row_size() || !t.is_contiguous() || t.view_src >= 0) return false;
        if (tx.ne[1] > 64 || !mmq_tc_supported(tw.ty, tx.ne[0], tw.ne[1], tx.ne[1]) || getenv("TLB_NO_TC") || getenv("TLB_MM_GENERIC")) return false;
        return true;
    };
    for (size_t i = 0; i < nn; i++) {
        if (dead[i]) continue;
        Tensor &A = g.tensors[g.nodes[i]];
        if (!eligible(A)) continue;
        int64_t tiles = (A.ne[0] + 127) / 128;
        int members = 1;
        const int wslot[3] = {0, 3, 5}, yslot[3] = {-1, 4, 6};
        for (size_t j = i + 1; j < nn && members < 3; j++) {
            const Tensor &B = g.tensors[g.nodes[j]];
            if (!eligible(B) || B.src[1] != A.src[1] || B.src[2] != A.src[2]) break;
            const int64_t tb = (B.ne[0] + 127) / 128;
            // a group stays within one wave of CTAs, or is big enough for the stream-K schedule (gate + up)
            if (tiles + tb > 148 && !mmq_tc_plan(g.tensors[A.src[1]].ne[0], (tiles + tb) * 128, g.tensors[A.src[1]].ne[1], 148).streamk) break;
            tiles += tb;
            A.src[wslot[members]] = B.src[0];
            A.src[yslot[members]] = g.nodes[j];
            dead[j] = 1;
            members++;
        }
        if (members > 1) A.op = "MUL_MAT_GROUP";
    }
    std::vector<int32_t> out;
    for (size_t i = 0; i < nn; i++)
        if (!dead[i]) out.push_back(g.nodes[i]);
    g.nodes.swap(out);
}

}  // namespace tlb
