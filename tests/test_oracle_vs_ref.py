"""The CPU oracle against the reference's own ggml build on larger seeded inputs at benchmark shapes
(runs where oracle/_ref exists; the committed golden vectors cover machines where it does not)."""
import numpy as np
import pytest

from oracle.bindings import F32, Q4_0, Q4_K, Q8_0

TYPES = [(Q8_0, "q8_0"), (Q4_0, "q4_0"), (Q4_K, "q4_K")]


@pytest.mark.parametrize("ty,name", TYPES)
@pytest.mark.parametrize("n", [4096, 14336])
def test_quantizers_match_reference(oracle, ref, ty, name, n):
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((16, n)) * 0.02).astype(np.float32)
    assert np.array_equal(oracle.quantize(ty, x), ref.quantize(ty, x))


def test_activation_quantizers_match_reference(oracle, ref):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((16, 4096)).astype(np.float32)
    assert np.array_equal(oracle.quantize(Q8_0, x), ref.act_q8_0(x))
    assert np.array_equal(oracle.quantize_q8_K(x), ref.act_q8_K(x))


@pytest.mark.parametrize("ty,name", TYPES)
def test_mul_mat_matches_cpu_backend(oracle, ref, ty, name):
    rng = np.random.default_rng(2)
    W = (rng.standard_normal((96, 4096)) * 0.02).astype(np.float32)
    X = rng.standard_normal((16, 4096)).astype(np.float32)
    Wq = ref.quantize(ty, W)
    g = ref.graph(128 << 20, 4)
    w = g.tensor(ty, [4096, 96], data=Wq)
    x = g.tensor(F32, [4096, 16], data=X)
    y = g.op("mul_mat", [w, x])
    g.compute([y])
    want = g.read(y).reshape(16, 96)
    got = oracle.mul_mat(ty, Wq, 4096, X)
    assert np.array_equal(got, want)
    # the gap to exact dequantized weights is what makes activation quantization part of parity
    exact = oracle.mul_mat(ty, Wq, 4096, X, dequant=True)
    gap = np.abs(exact - want).max() / np.abs(want).max()
    assert 1e-3 < gap < 3e-2


@pytest.mark.parametrize("ty", [3, 6, 7, 10, 11, 13, 14])
def test_decoders_match_reference(oracle, ref, ty):
    """q4_1 q5_0 q5_1 q2_K q3_K q5_K q6_K: bytes from the reference's quantizer, values from both dequantizers."""
    rng = np.random.default_rng(ty)
    x = (rng.standard_normal((12, 4096)) * 0.05).astype(np.float32)
    q = ref.quantize(ty, x)
    assert np.array_equal(oracle.dequantize(ty, q, 4096).view(np.uint32), ref.dequantize(ty, q, 4096).view(np.uint32))
