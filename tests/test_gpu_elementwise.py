"""The element-wise, normalisation, reduction and shape ops of the executor's table (SCALE FILL CLAMP LEAKY_RELU SQR SQRT
SIN COS LOG, the UNARY table, NORM, RMS_NORM, ADD SUB MUL DIV with broadcasting, SUM_ROWS, MEAN, REPEAT, CONCAT, ARANGE)
through one compiled program against the reference's own ggml CPU operators on the same inputs (the build of the
reference's vendored ggml under oracle/_ref). The reference runs the same comparison at 1e-4
(crates/tensorlisp/tests/native.rs:109-153); here copies, roundings and sign tests are compared for equality and everything
else to 1e-5 of max|want|. ggml's CPU GELU and GELU_QUICK go through an f16 lookup table, so those two are held to the
table's precision against ggml and to 1e-5 against the closed form."""
import math

import numpy as np
import pytest

from helpers import close
from tensorlisp_b200 import graph as G
from tensorlisp_b200.native import Native, NativeProgram
from test_graph_ir import build_both, elementwise_program

pytestmark = pytest.mark.gpu

EXACT = ("fill", "concat", "repeat", "arange", "unary abs", "unary sgn", "unary neg", "unary step", "unary relu", "unary floor",
         "unary ceil", "unary round", "unary trunc", "clamp", "leaky_relu")
TABLE = ("unary gelu", "unary gelu_quick")


def test_elementwise_ops_match_ggml(ref):
    named = []

    def prog(b):
        named.extend(elementwise_program(b))

    g, rg, pairs = build_both(ref, prog)
    rng = np.random.default_rng(11)
    inputs, host = {}, {}
    for a, b in pairs:
        T = g.tensors[a]
        if T.storage_kind == G.INPUT:
            data = (rng.standard_normal(T.ne[::-1]) * 1.5).astype(np.float32)
            inputs[T.storage_index] = data
            host[T.name] = data
            rg.write(b, data)
    for _, (a, _) in named:
        g.output(a)
    rg.compute([b for _, (_, b) in named])
    n = Native.load([])
    n.alloc_states([])
    prog_gpu = NativeProgram.compile(n, g, [(name, a) for name, (a, _) in named])
    for i, data in inputs.items():
        prog_gpu.set_input(i, data)
    prog_gpu.run()
    got = dict(prog_gpu.outputs())
    x = host["x"].astype(np.float64)
    closed = {"unary gelu": 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * x * (1.0 + 0.044715 * x * x))),
              "unary gelu_quick": x / (1.0 + np.exp(-1.702 * x))}
    for name, (a, b) in named:
        want = rg.read(b, np.float32)
        have = np.asarray(got[name], np.float32).reshape(want.shape)
        if name.startswith(EXACT):
            assert np.array_equal(have, want), name
        elif name in TABLE:
            close(have, want, 2e-3)
            close(have, closed[name].astype(np.float32).reshape(want.shape), 1e-5)
        else:
            err = close(have, want, 1e-5)
            print("%s: max error %.2e of max|want|" % (name, err / max(np.abs(want).max(), 1e-30)))
    prog_gpu.free()
    n.close()
    rg.close()


def indexing_inputs(g, pairs, rng):
    """Seeded inputs for indexing_program: masks with -inf holes (never a whole row), ids inside the tables, distinct
    destination rows per SET_ROWS column."""
    data = {}
    for a, _ in pairs:
        T = g.tensors[a]
        if T.storage_kind != G.INPUT:
            continue
        shape = T.ne[::-1]
        if T.name in ("mask16", "mask32"):
            m = rng.standard_normal(shape).astype(np.float32)
            m[rng.random(shape) < 0.3] = -np.inf
            m[..., 0] = 0.0
            v = m.astype(np.float16 if T.ty == G.F16 else np.float32)
        elif T.name == "table_i32":
            v = rng.integers(-1000, 1000, shape).astype(np.int32)
        elif T.name in ("ids1", "ids2"):
            v = rng.integers(0, 11, shape).astype(np.int32)
        elif T.name in ("at64", "at32"):
            v = np.stack([rng.permutation(11)[:4] for _ in range(int(np.prod(shape[:-1])))]).reshape(shape)
            v = v.astype(np.int64 if T.ty == G.I64 else np.int32)
        else:
            v = (rng.standard_normal(shape) * 2.0).astype(np.float16 if T.ty == G.F16 else np.float32)
        data[a] = v
    return data


def np_type(ty):
    return {G.F16: np.float16, G.I32: np.int32, G.I64: np.int64}.get(ty, np.float32)


def test_indexing_ops_match_ggml(ref):
    from test_graph_ir import indexing_program
    named = []

    def prog(b):
        named.extend(indexing_program(b))

    g, rg, pairs = build_both(ref, prog)
    data = indexing_inputs(g, pairs, np.random.default_rng(12))
    theirs = dict(pairs)
    for a, v in data.items():
        rg.write(theirs[a], v)
    for _, (a, _) in named:
        g.output(a)
    rg.compute([b for _, (_, b) in named])
    n = Native.load([])
    n.alloc_states([])
    prog_gpu = NativeProgram.compile(n, g, [(name, a) for name, (a, _) in named])
    for a, v in data.items():
        prog_gpu.set_input(g.tensors[a].storage_index, v)
    prog_gpu.run()
    got = dict(prog_gpu.outputs())
    for name, (a, b) in named:
        want = rg.read(b, np_type(g.tensors[a].ty)).astype(np.float32)
        have = np.asarray(got[name], np.float32).reshape(want.shape)
        if name.startswith("soft_max"):
            err = close(have, want, 1e-5)
            print("%s: max error %.2e of max|want|" % (name, err / max(np.abs(want).max(), 1e-30)))
        else:
            assert np.array_equal(have, want), name
    prog_gpu.free()
    n.close()
    rg.close()


def test_glu_variants_match_ggml(ref):
    """GLU in every form the executor takes (REGLU, GEGLU, SWIGLU, GEGLU_ERF, GEGLU_QUICK; one tensor cut in halves, straight
    and swapped, or two tensors) against ggml's CPU operator. GEGLU and GEGLU_QUICK read an f16 table on the CPU: those are
    held to the table's precision against ggml and to 1e-5 against the closed form."""
    from scipy.special import erf
    rng = np.random.default_rng(13)
    n, rows = 96, 7
    xu = (rng.standard_normal((rows, 2 * n)) * 2).astype(np.float32)
    a, u = np.ascontiguousarray(xu[:, :n]), np.ascontiguousarray(xu[:, n:])
    act = {
        "reglu": lambda x: np.maximum(x, 0),
        "geglu": lambda x: 0.5 * x * (1 + np.tanh(math.sqrt(2 / math.pi) * x * (1 + 0.044715 * x * x))),
        "swiglu": lambda x: x / (1 + np.exp(-x)),
        "geglu_erf": lambda x: 0.5 * x * (1 + erf(x / math.sqrt(2))),
        "geglu_quick": lambda x: x / (1 + np.exp(-1.702 * x)),
    }
    g, rg = G.Graph(), ref.graph(16 << 20, 1)
    t_xu, t_a, t_u = g.input(G.F32, [2 * n, rows], "xu"), g.input(G.F32, [n, rows], "a"), g.input(G.F32, [n, rows], "u")
    r_xu, r_a, r_u = rg.tensor(G.F32, [2 * n, rows], "xu", xu), rg.tensor(G.F32, [n, rows], "a", a), rg.tensor(G.F32, [n, rows], "u", u)
    cases = []
    for name, code in G.GLU_OPS.items():
        if name == "swiglu_oai":
            continue
        for form in ("halves", "swapped", "split"):
            if form == "split":
                ours, theirs = g.glu(t_a, name, b=t_u), rg.op("glu_split", [r_a, r_u], ints=[code])
                want64 = act[name](a.astype(np.float64)) * u
            else:
                sw = form == "swapped"
                ours, theirs = g.glu(t_xu, name, swapped=sw), rg.op("glu", [r_xu], ints=[code, int(sw)])
                want64 = act[name](u.astype(np.float64)) * a if sw else act[name](a.astype(np.float64)) * u
            g.output(ours)
            cases.append(("%s %s" % (name, form), ours, theirs, want64))
    rg.compute([c[2] for c in cases])
    n_dev = Native.load([])
    n_dev.alloc_states([])
    prog = NativeProgram.compile(n_dev, g, [(c[0], c[1]) for c in cases])
    for i, v in enumerate((xu, a, u)):
        prog.set_input(i, v)
    prog.run()
    got = dict(prog.outputs())
    for name, _, theirs, want64 in cases:
        want = rg.read(theirs).reshape(rows, n)
        have = np.asarray(got[name], np.float32).reshape(rows, n)
        if name.startswith(("geglu ", "geglu_quick")):
            close(have, want, 2e-3)
        else:
            close(have, want, 1e-5)
        close(have, want64.astype(np.float32), 1e-5)
    prog.free()
    n_dev.close()
    rg.close()


def test_copy_into_state_accumulates_in_graph_order():
    """cpy(add(state, x), state) followed by a read of the state, as the reference's `state_and_set_rows_persist_between_runs`
    does (crates/tensorlisp/tests/native.rs:437-468): the read comes after the write in graph order and sees the new sum; the
    sum survives runs and goes back to zero with reset_state."""
    from helpers import Model
    g = G.Graph()
    st = g.state(G.F32, [4], "sum")
    x = g.input(G.F32, [4], "x")
    g.cpy(g.add(st, x), st)
    g.output(g.scale(st, 1.0))
    m = Model(g, state_bytes=[16])
    rng = np.random.default_rng(14)
    total = np.zeros(4, np.float32)
    for _ in range(3):
        v = rng.standard_normal(4).astype(np.float32)
        total = total + v
        (got,) = m.run(v)
        assert np.array_equal(np.asarray(got, np.float32).reshape(4), total)
    m.native.reset_state()
    v = rng.standard_normal(4).astype(np.float32)
    (got,) = m.run(v)
    assert np.array_equal(np.asarray(got, np.float32).reshape(4), v)
    m.close()
