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
