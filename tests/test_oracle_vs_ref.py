"""The CPU oracle against the reference's own ggml build on larger seeded inputs at benchmark shapes
(runs where oracle/_ref exists; the committed golden vectors cover machines where it does not)."""
import numpy as np
import pytest

from oracle.bindings import BF16, F32, Q2_K, Q3_K, Q4_0, Q4_1, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0

TYPES = [(Q8_0, "q8_0"), (Q4_0, "q4_0"), (Q4_K, "q4_K")]
ALL_TARGETS = TYPES + [(Q4_1, "q4_1"), (Q5_0, "q5_0"), (Q5_1, "q5_1"), (Q2_K, "q2_K"), (Q3_K, "q3_K"), (Q5_K, "q5_K"), (Q6_K, "q6_K"),
                       (BF16, "bf16")]


@pytest.mark.parametrize("ty,name", ALL_TARGETS)
@pytest.mark.parametrize("n,scale", [(4096, 0.02), (14336, 0.02), (1024, 30.0)])
def test_quantizers_match_reference(oracle, ref, ty, name, n, scale):
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((16, n)) * scale).astype(np.float32)
    x[0, :256] = 0.0            # an all-zero super-block
    x[1, :32] = 0.25            # a constant block
    x[2, 256:512] = np.abs(x[2, 256:512])       # all positive: the minimum clamps to zero
    x[3, 7] = 1e4 * scale       # an outlier
    x[4, :16] = 1e-20           # below the all-zero threshold of the K-quant group search
    x[5, 32:64] = np.where(np.arange(32) % 2 == 0, 0.0, -0.0)     # zeros of both signs
    x[6, 32:64] = np.where(np.arange(32) % 2 == 0, -0.0, 0.0)
    assert np.array_equal(oracle.quantize(ty, x), ref.quantize(ty, x))


@pytest.mark.parametrize("ty,name", ALL_TARGETS)
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_quantizers_match_reference_on_varied_rows(oracle, ref, ty, name, seed):
    from helpers import varied_rows
    x = varied_rows(seed)
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


@pytest.mark.parametrize("ty,name", [t for t in ALL_TARGETS if t[1] != "bf16"])
def test_decoders_match_reference_on_varied_rows(oracle, ref, ty, name):
    """Every block type's decoder on the bytes the reference's quantizer gives for rows of very different character: the
    oracle's values must be ggml's, bit for bit."""
    from helpers import varied_rows
    x = varied_rows(3)
    q = ref.quantize(ty, x)
    mine, theirs = oracle.dequantize(ty, q, x.shape[1]), ref.dequantize(ty, q, x.shape[1])
    assert np.array_equal(mine.view(np.uint32), theirs.view(np.uint32))
