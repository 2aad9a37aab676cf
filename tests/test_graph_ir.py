"""The product's graph builder against ggml's own constructors (reference:
crates/tensorlisp/src/native_ir.rs:66-95 copies exactly these fields from a ggml_tensor)."""
import numpy as np
import pytest

from tensorlisp_b200 import graph as G


def build_both(ref, prog):
    """prog(b) drives a small recorder that issues each call to both builders."""
    g = G.Graph()
    rg = ref.graph(64 << 20, 1)
    pairs = []

    class B:
        def leaf(self, kind, ty, ne, name):
            a = getattr(g, kind)(ty, ne, name)
            b = rg.tensor(ty, ne, name)
            pairs.append((a, b))
            return (a, b)

        def op(self, ours, theirs, srcs, ours_args=(), ints=(), floats=(), **kw):
            a = getattr(g, ours)(*[s[0] if s is not None else None for s in srcs], *ours_args, **kw)
            b = rg.op(theirs, [s[1] if s is not None else None for s in srcs], ints, floats)
            pairs.append((a, b))
            return (a, b)

    prog(B())
    return g, rg, pairs


def compare(g, rg, pairs):
    back = {b: a for a, b in pairs}
    for a, b in pairs:
        T, info = g.tensors[a], rg.info(b)
        assert T.ty == info["ty"], (T.name, "type")
        assert list(T.ne) == info["ne"], (T.op, T.name, "ne", T.ne, info["ne"])
        assert list(T.nb) == info["nb"], (T.op, T.name, "nb", T.nb, info["nb"])
        assert T.op == info["op"], (T.name, T.op, info["op"])
        if T.op == "CUSTOM":  # slots 0,1 hold a function pointer (NULL), 4,5 the userdata
            assert T.op_params[2] == info["op_params"][2] and T.op_params[4:6] == info["op_params"][4:6]
        else:
            assert list(T.op_params) == info["op_params"], (T.op, T.name, T.op_params, info["op_params"])
        theirs_src = [back.get(s, -1) if s >= 0 else -1 for s in info["src"]]
        assert list(T.src) == theirs_src, (T.op, T.name, T.src, theirs_src)
        assert T.view_src == (back[info["view_src"]] if info["view_src"] >= 0 else -1), (T.op, T.name, "view_src")
        assert T.view_offs == info["view_offs"], (T.op, T.name, "view_offs")


def test_decoder_layer_ir_matches_ggml(ref):
    d, heads, kvh, hd, ffn, T = 256, 4, 2, 64, 512, 3

    def prog(b):
        x = b.leaf("input", G.F32, [d, T], "x")
        pos = b.leaf("input", G.I32, [T], "pos")
        wn = b.leaf("weight", G.F32, [d], "attn_norm")
        wq = b.leaf("weight", G.Q4_K, [d, heads * hd], "wq")
        wk = b.leaf("weight", G.Q8_0, [d, kvh * hd], "wk")
        wo = b.leaf("weight", G.Q4_0, [heads * hd, d], "wo")
        wg = b.leaf("weight", G.Q4_K, [d, ffn], "wg")
        wu = b.leaf("weight", G.Q4_K, [d, ffn], "wu")
        wd = b.leaf("weight", G.Q4_K, [ffn, d], "wd")
        n = b.op("rms_norm", "rms_norm", [x], (1e-5,), floats=[1e-5])
        h = b.op("mul", "mul", [n, wn])
        q = b.op("mul_mat", "mul_mat", [wq, h])
        k = b.op("mul_mat", "mul_mat", [wk, h])
        q3 = b.op("reshape", "reshape", [q], ([hd, heads, T],), ints=[hd, heads, T, 1])
        k3 = b.op("reshape", "reshape", [k], ([hd, kvh, T],), ints=[hd, kvh, T, 1])
        rope_o = (None, hd, 2, 0, 500000.0, 1.0, 0.0, 1.0, 32.0, 1.0)
        qr = b.op("rope_ext", "rope_ext", [q3, pos], rope_o, ints=[hd, 2, 0], floats=[500000.0, 1.0, 0.0, 1.0, 32.0, 1.0])
        kr = b.op("rope_ext", "rope_ext", [k3, pos], rope_o, ints=[hd, 2, 0], floats=[500000.0, 1.0, 0.0, 1.0, 32.0, 1.0])
        qh = b.op("cast", "cast", [qr], (G.F16,), ints=[G.F16])
        kh = b.op("cast", "cast", [kr], (G.F16,), ints=[G.F16])
        qp = b.op("permute", "permute", [qr], (0, 2, 1, 3), ints=[0, 2, 1, 3])
        kp = b.op("permute", "permute", [kr], (0, 2, 1, 3), ints=[0, 2, 1, 3])
        kc = b.op("cont", "cont", [kp])
        tr = b.op("transpose", "transpose", [x])
        trc = b.op("cont", "cont", [tr])
        a2 = b.op("reshape", "reshape", [qr], ([hd * heads, T],), ints=[hd * heads, T, 1, 1])
        o = b.op("mul_mat", "mul_mat", [wo, a2])
        x2 = b.op("add", "add", [x, o])
        gt = b.op("mul_mat", "mul_mat", [wg, x2])
        up = b.op("mul_mat", "mul_mat", [wu, x2])
        s = b.op("unary", "unary", [gt], ("silu",), ints=[10])
        m = b.op("mul", "mul", [s, up])
        g2 = b.op("glu", "glu_split", [gt, up], ints=[2], op="swiglu", b=None) if False else None
        dn = b.op("mul_mat", "mul_mat", [wd, m])
        x3 = b.op("add", "add", [x2, dn])
        sc = b.op("scale", "scale", [x3], (0.5, 0.25), floats=[0.5, 0.25])
        sm = b.op("soft_max_ext", "soft_max_ext", [sc, None], (0.125, 0.0), floats=[0.125, 0.0])
        am = b.op("argmax", "argmax", [sm])
        v = b.op("view", "view", [x3], ([d // 2, T], d * 4, 0, 0, d * 2), ints=[d // 2, T, 1, 1, d * 4, d * 4 * T, d * 4 * T, d * 2])

    g, rg, pairs = build_both(ref, prog)
    compare(g, rg, pairs)


def test_embedding_and_cache_ops_ir(ref):
    def prog(b):
        emb = b.leaf("weight", G.Q8_0, [256, 1000], "emb")
        ids = b.leaf("input", G.I32, [5], "ids")
        cache = b.leaf("state", G.F16, [64, 128], "cache")
        rows = b.leaf("input", G.F32, [64, 5], "rows")
        idx = b.leaf("input", G.I64, [5], "idx")
        e = b.op("get_rows", "get_rows", [emb, ids])
        s = b.op("set_rows", "set_rows", [cache, rows, idx])
        c = b.op("cpy", "cpy", [rows, b.op("view", "view", [cache], ([64, 5], 128, 0, 0, 0), ints=[64, 5, 1, 1, 128, 640, 640, 0])])

    g, rg, pairs = build_both(ref, prog)
    compare(g, rg, pairs)


def test_glu_and_paged_nodes_ir(ref):
    scale = 1.0 / np.sqrt(128.0)

    def prog(b):
        a = b.leaf("input", G.F32, [512, 4], "a")
        u = b.leaf("input", G.F32, [512, 4], "u")
        q = b.leaf("input", G.F16, [128, 8, 3], "q")
        kc = b.leaf("state", G.F16, [128 * 2 * 16, 10], "kc")
        vc = b.leaf("state", G.F16, [128 * 2 * 16, 10], "vc")
        tables = b.leaf("input", G.I32, [4, 3], "tables")
        lens = b.leaf("input", G.I32, [3], "lens")
        key = b.leaf("input", G.F16, [256, 3], "key")
        val = b.leaf("input", G.F16, [256, 3], "val")
        slots = b.leaf("input", G.I32, [6], "slots")
        g1 = b.op("glu", "glu", [a], ("swiglu", False), ints=[2, 0])
        g2 = b.op("glu", "glu", [a], ("geglu", True), ints=[1, 1])
        ud1 = G.Graph.paged_userdata(1, 2, 16, 64, scale)
        ud2 = G.Graph.paged_userdata(2, 2, 16, 1, 1.0)
        p = b.op("paged_attention", "custom", [q, kc, vc, tables, lens], (16, 64, scale, 2), ints=[G.F16, 128, 8, 3, 1, ud1])
        w = b.op("paged_cache_write", "custom", [key, val, kc, vc, slots], (16, 2), ints=[G.F16, 1, 1, 1, 1, ud2])

    g, rg, pairs = build_both(ref, prog)
    compare(g, rg, pairs)
    g2 = G.Graph()
    a = g2.input(G.F32, [512, 4], "a")
    u = g2.input(G.F32, [512, 4], "u")
    t = g2.glu(a, "swiglu", b=u)
    assert g2.tensors[t].ne == [512, 4, 1, 1] and g2.tensors[t].src[:2] == [a, u]


def image_ops_program(b):
    """Every image-op constructor once or more, with ggml's own constructor beside it; returns (name, node pair) list."""
    x = b.leaf("input", G.F32, [10, 12, 4, 2], "img")
    k16 = b.leaf("input", G.F16, [3, 3, 4, 8], "kernel")
    kdw = b.leaf("input", G.F32, [3, 2, 1, 4], "dw_kernel")
    x1 = b.leaf("input", G.F32, [50, 6, 3], "signal")
    k1 = b.leaf("input", G.F16, [5, 6, 7], "kernel_1d")
    out = []
    out.append(("im2col 2d f16", b.op("im2col", "im2col", [k16, x], (1, 2, 1, 0, 1, 2, True, G.F16), ints=[1, 2, 1, 0, 1, 2, 1, G.F16])))
    out.append(("im2col 2d f32", b.op("im2col", "im2col", [k16, x], (2, 1, 0, 1, 1, 1, True, G.F32), ints=[2, 1, 0, 1, 1, 1, 1, G.F32])))
    out.append(("im2col 1d", b.op("im2col", "im2col", [k1, x1], (2, 0, 3, 0, 2, 0, False, G.F16), ints=[2, 0, 3, 0, 2, 0, 0, G.F16])))
    for mode in (0, 1, 2, 1 | (1 << 8), 2 | (1 << 8), 1 | (1 << 9)):
        out.append(("upscale mode %d" % mode, b.op("interpolate", "interpolate", [x], (23, 17, 4, 2, mode), ints=[23, 17, 4, 2, mode])))
    out.append(("downscale antialias", b.op("interpolate", "interpolate", [x], (4, 5, 4, 2, 1 | (1 << 9)), ints=[4, 5, 4, 2, 1 | (1 << 9)])))
    out.append(("upscale x2", b.op("interpolate", "interpolate", [x], (20, 24, 4, 2, 0), ints=[20, 24, 4, 2, 0])))
    out.append(("pool max", b.op("pool_2d", "pool_2d", [x], (0, 3, 2, 2, 2, 1.0, 0.0), ints=[0, 3, 2, 2, 2], floats=[1.0, 0.0])))
    out.append(("pool avg", b.op("pool_2d", "pool_2d", [x], (1, 2, 2, 2, 2, 0.0, 0.0), ints=[1, 2, 2, 2, 2], floats=[0.0, 0.0])))
    out.append(("conv_2d_dw", b.op("conv_2d_dw", "conv_2d_dw", [kdw, x], (1, 2, 1, 1, 2, 1), ints=[1, 2, 1, 1, 2, 1])))
    out.append(("pad_ext", b.op("pad_ext", "pad_ext", [x], (1, 2, 0, 3, 2, 0, 1, 1), ints=[1, 2, 0, 3, 2, 0, 1, 1])))
    out.append(("pad_reflect_1d", b.op("pad_reflect_1d", "pad_reflect_1d", [x], (3, 5), ints=[3, 5])))
    return out


def elementwise_program(b):
    """The element-wise, normalisation, reduction and shape ops of the executor's table (crates/kernels/src/cuda/lower.rs:177-213),
    each with ggml's own constructor beside it: what the reference's test `elementwise_norms_and_reductions` runs
    (crates/tensorlisp/tests/native.rs:109-153) and the rest of the unary table. Returns (name, node pair) list."""
    x = b.leaf("input", G.F32, [24, 7, 3], "x")
    y = b.leaf("input", G.F32, [24, 7, 3], "y")
    row = b.leaf("input", G.F32, [24, 1, 3], "row")     # broadcasts over dimension 1
    out = []
    out.append(("norm", b.op("norm", "norm", [x], (1e-6,), floats=[1e-6])))
    out.append(("rms_norm", b.op("rms_norm", "rms_norm", [x], (1e-5,), floats=[1e-5])))
    for name, code in G.UNARY_OPS.items():
        if name != "xielu":
            out.append(("unary " + name, b.op("unary", "unary", [x], (name,), ints=[code])))
    out.append(("scale", b.op("scale", "scale", [x], (0.5, 3.0), floats=[0.5, 3.0])))
    sq = b.op("sqr", "sqr", [x])
    out.append(("sqr", sq))
    out.append(("sqrt", b.op("sqrt", "sqrt", [sq])))
    out.append(("log", b.op("log", "log", [b.op("scale", "scale", [sq], (1.0, 0.1), floats=[1.0, 0.1])])))
    out.append(("sin", b.op("sin", "sin", [x])))
    out.append(("cos", b.op("cos", "cos", [y])))
    out.append(("leaky_relu", b.op("leaky_relu", "leaky_relu", [x], (0.1,), floats=[0.1])))
    out.append(("fill", b.op("fill", "fill", [x], (2.5,), floats=[2.5])))
    # clamp works in place: it gets a copy of its own to change
    out.append(("clamp", b.op("clamp", "clamp", [b.op("scale", "scale", [x], (1.0, 0.0), floats=[1.0, 0.0])], (-0.5, 0.7), floats=[-0.5, 0.7])))
    ey = b.op("scale", "scale", [b.op("unary", "unary", [y], ("exp",), ints=[G.UNARY_OPS["exp"]])], (1.0, 2.0), floats=[1.0, 2.0])
    out.append(("arith", b.op("div", "div", [b.op("sub", "sub", [b.op("mul", "mul", [x, y]), sq]), ey])))
    out.append(("add broadcast", b.op("add", "add", [x, row])))
    out.append(("mul broadcast", b.op("mul", "mul", [x, row])))
    out.append(("sum_rows", b.op("sum_rows", "sum_rows", [x])))
    out.append(("mean", b.op("mean", "mean", [x])))
    out.append(("repeat", b.op("repeat", "repeat", [row, x])))
    for dim in (0, 1, 2):
        out.append(("concat %d" % dim, b.op("concat", "concat", [x, y], (dim,), ints=[dim])))
    out.append(("arange", b.op("arange", "arange", [], (1.0, 10.0, 1.5), floats=[1.0, 10.0, 1.5])))
    return out


def indexing_program(b):
    """SOFT_MAX with f16 and f32 masks, per-head masks and ALiBi slopes; GET_ROWS from f32 / f16 / i32 tables with batched
    ids; SET_ROWS into f32 and f16 destinations with i64 and i32 ids broadcast over the batch; copies of permuted and
    transposed sources. Returns (name, node pair) list."""
    out = []
    s = b.leaf("input", G.F32, [40, 9, 6, 2], "scores")                 # [keys, queries, heads, batch]
    m16 = b.leaf("input", G.F16, [40, 32, 1, 1], "mask16")             # one mask for all heads, padded rows
    m32 = b.leaf("input", G.F32, [40, 9, 6, 1], "mask32")              # a mask per head
    out.append(("soft_max plain", b.op("soft_max_ext", "soft_max_ext", [s, None], (0.7, 0.0), floats=[0.7, 0.0])))
    out.append(("soft_max f16 mask", b.op("soft_max_ext", "soft_max_ext", [s, m16], (0.3, 0.0), floats=[0.3, 0.0])))
    out.append(("soft_max f32 mask per head", b.op("soft_max_ext", "soft_max_ext", [s, m32], (1.0, 0.0), floats=[1.0, 0.0])))
    out.append(("soft_max alibi", b.op("soft_max_ext", "soft_max_ext", [s, m16], (0.5, 8.0), floats=[0.5, 8.0])))
    t32 = b.leaf("input", G.F32, [16, 11, 3], "table32")
    t16 = b.leaf("input", G.F16, [16, 11, 3], "table16")
    ti = b.leaf("input", G.I32, [16, 11], "table_i32")
    ids2 = b.leaf("input", G.I32, [5, 3], "ids2")                       # one list of ids per batch entry of the table
    ids1 = b.leaf("input", G.I32, [4], "ids1")
    out.append(("get_rows f32 batched", b.op("get_rows", "get_rows", [t32, ids2])))
    out.append(("get_rows f16 batched", b.op("get_rows", "get_rows", [t16, ids2])))
    out.append(("get_rows i32", b.op("get_rows", "get_rows", [ti, ids1])))
    rows = b.leaf("input", G.F32, [16, 4, 3], "rows")
    at64 = b.leaf("input", G.I64, [4, 1], "at64")                       # the same rows of every batch entry
    at32 = b.leaf("input", G.I32, [4, 3], "at32")
    d32 = b.op("scale", "scale", [t32], (1.0, 0.0), floats=[1.0, 0.0])   # destinations that the node may write
    d16 = b.op("cast", "cast", [t32], (G.F16,), ints=[G.F16])
    w32 = b.op("set_rows", "set_rows", [d32, rows, at64])
    w16 = b.op("set_rows", "set_rows", [d16, rows, at32])
    out.append(("set_rows f32", b.op("scale", "scale", [w32], (1.0, 0.0), floats=[1.0, 0.0])))
    out.append(("set_rows f16", b.op("cast", "cast", [w16], (G.F32,), ints=[G.F32])))
    out.append(("cont permuted", b.op("cont", "cont", [b.op("permute", "permute", [s], (2, 0, 1, 3), ints=[2, 0, 1, 3])])))
    out.append(("cont transposed f16", b.op("cont", "cont", [b.op("transpose", "transpose", [t16])])))
    out.append(("cast permuted", b.op("cast", "cast", [b.op("permute", "permute", [t32], (1, 0, 2, 3), ints=[1, 0, 2, 3])], (G.F16,), ints=[G.F16])))
    return out


def test_indexing_op_ir_matches_ggml(ref):
    g, rg, pairs = build_both(ref, indexing_program)
    compare(g, rg, pairs)
    rg.close()


def test_elementwise_op_ir_matches_ggml(ref):
    g, rg, pairs = build_both(ref, elementwise_program)
    compare(g, rg, pairs)
    rg.close()


def test_image_op_ir_matches_ggml(ref):
    g, rg, pairs = build_both(ref, image_ops_program)
    compare(g, rg, pairs)
    rg.close()
