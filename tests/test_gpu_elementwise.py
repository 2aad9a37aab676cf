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
