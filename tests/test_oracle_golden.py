"""The CPU oracle (oracle/oracle.c) against the golden vectors generated from the reference's own
ggml build (tests/golden/make_golden.py). This is what pins the oracle: integer/byte outputs must be
identical, float outputs identical up to the last-bit effects stated per case."""
import os

import numpy as np
import pytest

from oracle.bindings import F32, Q4_0, Q4_K, Q8_0

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
TYPES = [(Q8_0, "q8_0"), (Q4_0, "q4_0"), (Q4_K, "q4_K")]


@pytest.mark.parametrize("ty,name", TYPES)
def test_weight_quantizers_bit_exact(oracle, ty, name):
    got = oracle.quantize(ty, G["quant_x"])
    assert np.array_equal(got, G["quant_" + name])
    assert np.array_equal(oracle.dequantize(ty, got, 512), G["dequant_" + name])


def test_activation_quantizers_bit_exact(oracle):
    assert np.array_equal(oracle.quantize(Q8_0, G["act_x"]), G["act_q8_0"])
    got = oracle.quantize_q8_K(G["act_x"]).reshape(-1, 292)
    want = G["act_q8_K"].reshape(-1, 292)
    # the reference leaves bsums of an all-zero block unwritten: compare d and qs there, everything elsewhere
    zero = np.all(want[:, 4:260] == 0, axis=1) & np.all(want[:, :4] == 0, axis=1)
    assert np.array_equal(got[~zero], want[~zero])
    assert np.array_equal(got[zero][:, :260], want[zero][:, :260])


@pytest.mark.parametrize("ty,name", TYPES)
def test_mul_mat_identical(oracle, ty, name):
    W = oracle.quantize(ty, G["mm_w"])
    y = oracle.mul_mat(ty, W, 512, G["mm_x"])
    assert np.array_equal(y, G["mm_y_" + name])


def test_row_ops(oracle):
    x, w, u = G["row_x"], G["row_w"], G["row_u"]
    assert np.array_equal(oracle.rms_norm(x, 1e-5, w), G["row_rms_mul"])
    assert np.array_equal(oracle.rms_norm(x, 1e-6), G["row_rms"])
    # the reference's SiLU runs a vectorised exp approximation (ggml-cpu/vec.cpp, SSE2 path): a few ulp
    np.testing.assert_allclose(oracle.silu_mul(x, u), G["row_silu_mul"], rtol=2e-6, atol=1e-30)
    np.testing.assert_allclose(oracle.silu_mul(x, u), G["row_swiglu"], rtol=2e-6, atol=1e-30)
    np.testing.assert_allclose(oracle.soft_max(x, 0.25), G["row_softmax"], rtol=2e-6, atol=1e-12)
    assert np.array_equal(oracle.argmax(x), G["row_argmax"])
    assert np.array_equal(oracle.argmax(G["ties_x"]), G["ties_argmax"])
    assert list(G["ties_argmax"]) == [29, 39, 39]


def test_rope(oracle):
    x, pos = G["rope_x"], G["rope_pos"]
    np.testing.assert_allclose(oracle.rope(x, pos, 128, 2, 500000.0), G["rope_neox"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(oracle.rope(x, pos, 128, 0, 500000.0), G["rope_normal"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(oracle.rope(x, pos, 64, 2, 10000.0), G["rope_neox_partial"], rtol=0, atol=2e-6)


def test_get_rows(oracle):
    tab = oracle.quantize(Q8_0, G["emb_table"])
    assert np.array_equal(oracle.get_rows(Q8_0, tab, 256, G["emb_ids"]), G["emb_rows"])


def test_attention_decode(oracle):
    q = G["att_q"]
    ks = [G["att_k%d" % s] for s in range(3)]
    vs = [G["att_v%d" % s] for s in range(3)]
    _, out32 = oracle.attention_decode(q, ks, vs, 2, 1.0 / np.sqrt(128.0))
    want = G["att_out"]
    assert np.abs(out32 - want).max() <= 2e-5 * np.abs(want).max()


DEC = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_decoders.npz"))
DECODED = [(3, "q4_1"), (6, "q5_0"), (7, "q5_1"), (10, "q2_K"), (11, "q3_K"), (13, "q5_K"), (14, "q6_K")]


@pytest.mark.parametrize("ty,name", DECODED)
def test_decoders_of_the_other_block_types(oracle, ty, name):
    """The bytes are the reference's (ggml_quantize_chunk); the oracle's dequantizer must give ggml's values, bit for bit."""
    q = DEC["quant_" + name]
    assert q.shape[1] == oracle.row_size(ty, 512)
    assert np.array_equal(oracle.dequantize(ty, q, 512).view(np.uint32), DEC["dequant_" + name].view(np.uint32))
    # and the oracle's quantizer gives the reference's bytes for the same rows
    assert np.array_equal(oracle.quantize(ty, DEC["x"]), q)
    # the values are what the type can hold of x: a few percent of the row scale at most (2- and 3-bit types are coarse)
    x, y = DEC["x"], DEC["dequant_" + name]
    assert np.abs(x - y).max() <= 0.5 * np.abs(x).max()
