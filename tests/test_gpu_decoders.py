"""The block types the executor reads through its element decoders (q4_1 q5_0 q5_1 q2_K q3_K q5_K q6_K; reference
decoders crates/kernels/src/cuda/native/common.cuh:169-263): dequantizing copy, embedding lookup and mul_mat at the
reference's batch grid N in {1, 3, 5, 8, 9, 40} (crates/tensorlisp/tests/native.rs:72-106). The bytes are the
reference's own quantizer output (tests/golden/golden_decoders.npz); decoded values must be ggml's bit for bit, and
mul_mat is compared with the exact dequantized weights times the activations, the reference test's own comparison
(its bar: 4e-3 of the scale)."""
import os

import numpy as np
import pytest

from helpers import Model, close
from tensorlisp_b200 import graph as G

pytestmark = pytest.mark.gpu
DEC = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_decoders.npz"))
TYPES = [(G.Q4_1, "q4_1"), (G.Q5_0, "q5_0"), (G.Q5_1, "q5_1"), (G.Q2_K, "q2_K"), (G.Q3_K, "q3_K"), (G.Q5_K, "q5_K"), (G.Q6_K, "q6_K")]


@pytest.mark.parametrize("ty,name", TYPES)
def test_dequantizing_copy_and_lookup(ty, name):
    q, want = DEC["quant_" + name], DEC["dequant_" + name]
    rows = q.shape[0]
    ids = np.array([5, 0, rows - 1, 9, 9], np.int32)
    g = G.Graph()
    w = g.weight(ty, [512, rows], "w")
    ti = g.input(G.I32, [len(ids)], "ids")
    a = g.output(g.cast(w, G.F32, "values"))
    b = g.output(g.get_rows(w, ti, "rows"))
    m = Model(g, [q])
    got_a, got_b = m.run(ids)
    m.close()
    assert np.array_equal(got_a.reshape(rows, 512).view(np.uint32), want.view(np.uint32))
    assert np.array_equal(got_b.reshape(len(ids), 512).view(np.uint32), want[ids].view(np.uint32))


@pytest.mark.parametrize("ty,name", TYPES)
def test_mul_mat_by_type_and_batch(oracle, ty, name):
    q = DEC["quant_" + name]
    rows = q.shape[0]
    rng = np.random.default_rng(ty)
    worst = 0.0
    for n in (1, 3, 5, 8, 9, 40):
        x = rng.standard_normal((n, 512)).astype(np.float32)
        g = G.Graph()
        w = g.weight(ty, [512, rows], "w")
        tx = g.input(G.F32, [512, n], "x")
        y = g.output(g.mul_mat(w, tx, "y"))
        m = Model(g, [q])
        (got,) = m.run(x)
        m.close()
        want = oracle.mul_mat(ty, q, 512, x, dequant=True)
        worst = max(worst, close(got.reshape(n, rows), want, 4e-3))
    assert worst <= 1e-4 * np.abs(want).max() + 1e-6    # f32 accumulation against the oracle's f64: far inside the bar
