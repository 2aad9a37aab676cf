"""GPU row quantizers through the C ABI (tlb_quantize_rows) against the oracle and the golden
vectors: bit-exact bytes (reference: crates/tensorlisp/src/dtype.rs:98-124 -> ggml_quantize_chunk)."""
import os

import numpy as np
import pytest

from oracle.bindings import BF16, Q2_K, Q3_K, Q4_0, Q4_1, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0
from tensorlisp_b200.native import TlbError, quantize_rows

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
DEC = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_decoders.npz"))
TYPES = [(Q8_0, "q8_0"), (Q4_0, "q4_0"), (Q4_K, "q4_K")]
MORE = [(Q4_1, "q4_1"), (Q5_0, "q5_0"), (Q5_1, "q5_1"), (Q2_K, "q2_K"), (Q3_K, "q3_K"), (Q5_K, "q5_K"), (Q6_K, "q6_K")]


@pytest.mark.parametrize("ty,name", TYPES)
def test_golden_bytes(native, ty, name):
    got = quantize_rows(native, ty, G["quant_x"])
    assert np.array_equal(got, G["quant_" + name])


@pytest.mark.parametrize("ty,name", MORE)
def test_golden_bytes_of_the_other_block_types(native, ty, name):
    """The reference's own bytes (ggml_quantize_chunk) for seeded random rows and edge-case rows: all-zero and constant
    blocks, an outlier, tiny and huge magnitudes."""
    got = quantize_rows(native, ty, DEC["x"])
    assert np.array_equal(got, DEC["quant_" + name])


@pytest.mark.parametrize("ty,name", TYPES + MORE + [(BF16, "bf16")])
@pytest.mark.parametrize("shape,scale,seed", [((64, 4096), 0.02, 0), ((8, 14336), 0.02, 3), ((33, 256), 1.0, 4), ((5, 1024), 50.0, 5)])
def test_against_oracle(native, oracle, ty, name, shape, scale, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(shape) * scale).astype(np.float32)
    x[0, :256] = 0.0          # an all-zero super-block
    x[-1, :32] = 0.25         # a constant block
    x[1, :256] = np.abs(x[1, :256])        # all positive: the block minimum clamps to zero in the K-quants
    x[2, 5] = 3e3 * scale     # an outlier
    x[3, :16] = 1e-20         # a group below the all-zero threshold of the K-quant searches
    x[4, 32:64] = np.where(np.arange(32) % 2 == 0, 0.0, -0.0)   # zeros of both signs (first minimum / maximum wins)
    got, want = quantize_rows(native, ty, x), oracle.quantize(ty, x)
    if ty == BF16:
        got, want = got.view(np.uint8), want.view(np.uint8)
    assert np.array_equal(got.reshape(want.shape), want)


@pytest.mark.parametrize("ty,name", TYPES + MORE + [(BF16, "bf16")])
def test_varied_rows(native, oracle, ty, name):
    """Rows of very different character (scales from 1e-6 to 1e4, heavy tails, sparse, one-sided, constant, ramps, zero
    blocks inside noise, f16's limits, many exact ties): the bytes must still be the oracle's, which the CPU suite holds
    against the reference's own quantizers on the same rows."""
    from helpers import varied_rows
    for seed in (0, 1, 2):
        x = varied_rows(seed)
        got, want = quantize_rows(native, ty, x), oracle.quantize(ty, x)
        assert np.array_equal(got.view(np.uint8).reshape(want.shape), want), (name, seed)


def test_config1_matrix_q8_0_bit_exact(native, oracle):
    """benchmark config 1: 4096x4096 N(0, 0.02) seed 0 -> Q8_0."""
    x = (np.random.default_rng(0).standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    got = quantize_rows(native, Q8_0, x)
    assert got.shape == (4096, 4352)
    assert np.array_equal(got, oracle.quantize(Q8_0, x))


def test_q4_K_full_rows_and_idempotence(native, oracle):
    """Size-independent properties at full row lengths: quantizing the dequantized output again
    reproduces the same codes' values (dequant is a fixed point of quantize o dequant for Q8_0)."""
    x = (np.random.default_rng(7).standard_normal((512, 14336)) * 0.02).astype(np.float32)
    q = quantize_rows(native, Q4_K, x)
    assert np.array_equal(q, oracle.quantize(Q4_K, x))
    q8 = quantize_rows(native, Q8_0, x)
    d8 = oracle.dequantize(Q8_0, q8, 14336)
    assert np.array_equal(oracle.dequantize(Q8_0, quantize_rows(native, Q8_0, d8), 14336), d8)
    # the reconstruction error stays within half a quantization step of each block, plus the f16
    # rounding of the block scale (127 codes * 2^-11 relative)
    step = np.abs(x).reshape(512, -1, 32).max(axis=2) / 127
    assert np.all(np.abs(d8 - x).reshape(512, -1, 32).max(axis=2) <= step * (0.5 + 127 / 2048) + 1e-7)


def test_empty_and_bad_rows(native):
    assert quantize_rows(native, Q8_0, np.zeros((0, 64), np.float32)).shape == (0, 68)
    with pytest.raises(TlbError) as e:
        quantize_rows(native, Q4_K, np.zeros((2, 100), np.float32))
    assert "multiple of the block size" in str(e.value)
    with pytest.raises(TlbError) as e:
        quantize_rows(native, 20, np.zeros((2, 256), np.float32))  # iq4_nl is not implemented
    assert "not implemented" in str(e.value)


def test_quantize_file_like_tl_quantize(native, oracle, tmp_path):
    """`tl quantize` on the GPU: the weights the program feeds into MUL_MAT / GET_ROWS (seen through views) become Q4_K,
    bit-exact with the oracle; a matrix the graph also ADDs, the 1-D norm, the ragged matrix, the program and the
    asset are carried over, each with the reference's reason (crates/tensorlisp-cli/src/quantize.rs:148-191). An
    already quantized tensor is converted only with `requantize`, from its dequantized values."""
    from tensorlisp_b200 import graph as G
    from tensorlisp_b200.gguf import GgufFile, GgufWriter, quantize_file
    rng = np.random.default_rng(8)
    w = (rng.standard_normal((40, 1024)) * 0.02).astype(np.float32)
    emb = (rng.standard_normal((64, 1024)) * 0.02).astype(np.float32)
    bias_like = rng.standard_normal((40, 1024)).astype(np.float32)
    ragged = rng.standard_normal((4, 100)).astype(np.float32)
    w8 = oracle.quantize(G.Q8_0, w)
    src, dst = str(tmp_path / "f32.gguf"), str(tmp_path / "q4k.gguf")
    out = GgufWriter()
    out.set_program("(define (f x) x)")
    out.set_asset("a.bin", b"abc")
    out.add_tensor("norm", G.F32, [1024], np.ones(1024, np.float32))
    out.add_tensor("W", G.F32, [1024, 40], w)
    out.add_tensor("emb", G.F32, [1024, 64], emb)
    out.add_tensor("added", G.F32, [1024, 40], bias_like)
    out.add_tensor("ragged", G.F32, [100, 4], ragged)
    out.add_tensor("W8", G.Q8_0, [1024, 40], w8)
    out.add_tensor("unused", G.F32, [1024, 40], w)
    out.write(src)
    # the program: y = W . norm(emb[ids]) + W8 . h, with `added` used by an ADD as well as by a MUL_MAT
    g = G.Graph()
    tn = g.weight(G.F32, [1024], "norm")
    tw = g.weight(G.F32, [1024, 40], "W")
    te = g.weight(G.F32, [1024, 64], "emb")
    ta = g.weight(G.F32, [1024, 40], "added")
    t8 = g.weight(G.Q8_0, [1024, 40], "W8")
    ids = g.input(G.I32, [3], "ids")
    h = g.mul(g.rms_norm(g.get_rows(te, ids), 1e-5), tn)
    y = g.add(g.mul_mat(g.reshape(tw, [1024, 40]), h), g.mul_mat(t8, h))       # W is seen through a view op
    y = g.add(y, g.mul_mat(ta, h))
    g.output(g.add(g.sum_rows(ta), g.sum_rows(ta)))
    g.output(y)
    rep = {r["name"]: r for r in quantize_file(native, src, dst, G.Q4_K, graphs=[g])}
    assert rep["W"]["kept_because"] is None and rep["emb"]["kept_because"] is None
    assert rep["norm"]["kept_because"] == "used by MUL (source 1); only matmul/get-rows weights are quantized"
    assert rep["added"]["kept_because"] == "used by SUM_ROWS (source 0); only matmul/get-rows weights are quantized"
    assert rep["ragged"]["kept_because"] == "not used by the program"
    assert rep["unused"]["kept_because"] == "not used by the program"
    assert rep["W8"]["kept_because"] == "already quantized (use --requantize)"
    f = GgufFile(dst)
    assert f.program() == "(define (f x) x)" and f.assets() == {"a.bin": b"abc"}
    assert [(t.name, t.ty) for t in f.tensors] == [("norm", G.F32), ("W", G.Q4_K), ("emb", G.Q4_K), ("added", G.F32), ("ragged", G.F32),
                                                   ("W8", G.Q8_0), ("unused", G.F32)]
    assert np.array_equal(f.tensor_bytes(1), oracle.quantize(G.Q4_K, w).reshape(-1))
    assert np.array_equal(f.tensor_bytes(4).view(np.float32).reshape(4, 100), ragged)
    f.close()
    # without a graph: by name, rank and size only
    rep = {r["name"]: r for r in quantize_file(native, src, dst, G.Q4_K, exclude=["un*"], requantize=True)}
    assert rep["norm"]["kept_because"] == "1-D (use --include-1d)"
    assert rep["ragged"]["kept_because"] == "fewer than 1024 elements"
    assert rep["unused"]["kept_because"] == "excluded by un*"
    assert rep["added"]["kept_because"] is None and rep["W8"]["kept_because"] is None
    f = GgufFile(dst)
    i8 = [t.name for t in f.tensors].index("W8")
    assert f.tensors[i8].ty == G.Q4_K
    assert np.array_equal(f.tensor_bytes(i8), oracle.quantize(G.Q4_K, oracle.dequantize(G.Q8_0, w8, 1024)).reshape(-1))
    f.close()


def test_convert_safetensors_like_tl_convert(native, oracle, tmp_path):
    """`tl convert --dtype q4_K` on the GPU (crates/tensorlisp-cli/src/convert.rs): matrices become Q4_K (one, by a --type
    rule, Q8_0), bit-exact with the oracle from the f32 values of their f32 / f16 / bf16 sources; the 1-D norm stays f32 and
    takes its --offset; integers become i32; a small f64 matrix becomes f16; names are rewritten; program and metadata are
    stored."""
    from helpers import write_safetensors
    from tensorlisp_b200 import graph as G
    from tensorlisp_b200.gguf import GgufFile, convert_safetensors
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((40, 1024)) * 0.02).astype(np.float32)
    h = rng.standard_normal((8, 512)).astype(np.float16)
    b = (rng.standard_normal((4, 256)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    norm = rng.standard_normal(1024).astype(np.float32)
    ids = np.array([3, 1, 4, 1, 5, 9], np.int64)
    small = rng.standard_normal((4, 32))
    src, dst = str(tmp_path / "m.safetensors"), str(tmp_path / "m.gguf")
    write_safetensors(src, {"model.w": w, "model.f16m": h, "model.b": ("BF16", b), "model.norm.weight": norm, "model.ids": ids, "model.small": small})
    rep = convert_safetensors(native, src, dst, "q4_K", program="(define (f x) x)", meta=["general.name=tiny"], strip_prefix=["model."],
                              types=["*f16m*=q8_0"], offset=["*norm.weight=1"])
    assert [t["to"] for t in rep["tensors"]] == ["q4_K", "q8_0", "q4_K", "f32", "i32", "f16"] and rep["skipped"] == []
    f = GgufFile(dst)
    got = {t.name: (t, f.tensor_bytes(i)) for i, t in enumerate(f.tensors)}
    assert set(got) == {"w", "f16m", "b", "norm.weight", "ids", "small"}
    assert got["w"][0].ty == G.Q4_K and got["w"][0].ne[:2] == [1024, 40]
    assert np.array_equal(np.frombuffer(got["w"][1], np.uint8), oracle.quantize(Q4_K, w).reshape(-1))
    assert np.array_equal(np.frombuffer(got["f16m"][1], np.uint8), oracle.quantize(Q8_0, h.astype(np.float32)).reshape(-1))
    bf = (b.astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(np.frombuffer(got["b"][1], np.uint8), oracle.quantize(Q4_K, bf).reshape(-1))
    assert np.array_equal(np.frombuffer(got["norm.weight"][1], np.float32), norm + np.float32(1))
    assert np.array_equal(np.frombuffer(got["ids"][1], np.int32), ids.astype(np.int32))
    assert np.array_equal(np.frombuffer(got["small"][1], np.float16), small.astype(np.float32).astype(np.float16).reshape(-1))
    assert f.program() == "(define (f x) x)" and f.kv["general.name"][1] == "tiny"
    f.close()


def test_a_converted_file_loads_and_runs(native, oracle, tmp_path):
    """safetensors -> `tl convert --dtype q8_0` on the GPU -> GGUF on disk -> Native.load_gguf -> a program over the stored
    weights: the embedding lookup returns the dequantized rows and the projection agrees with the oracle on the file's bytes."""
    from helpers import close, write_safetensors
    from tensorlisp_b200 import graph as G
    from tensorlisp_b200.gguf import convert_safetensors
    from tensorlisp_b200.native import Native, NativeProgram
    rng = np.random.default_rng(10)
    emb = (rng.standard_normal((50, 256)) * 0.1).astype(np.float32)
    proj = (rng.standard_normal((96, 256)) * 0.02).astype(np.float32)
    src, dst = str(tmp_path / "m.safetensors"), str(tmp_path / "m.gguf")
    write_safetensors(src, {"embed.weight": emb, "proj.weight": proj})
    convert_safetensors(native, src, dst, "q8_0", program="(define (f ids) ids)")
    n, f = Native.load_gguf(dst)
    assert [t.name for t in f.tensors] == ["embed.weight", "proj.weight"] and all(t.ty == G.Q8_0 for t in f.tensors)
    n.alloc_states([])
    g = G.Graph()
    we = g.weight(G.Q8_0, [256, 50], "embed.weight")
    wp = g.weight(G.Q8_0, [256, 96], "proj.weight")
    ids = g.input(G.I32, [4], "ids")
    rows = g.get_rows(we, ids, "rows")
    g.output(rows)
    g.output(g.mul_mat(wp, rows, "scores"))
    prog = NativeProgram.compile(n, g)
    which = np.array([7, 0, 49, 7], np.int32)
    prog.set_input(0, which)
    prog.run()
    out = dict(prog.outputs())
    eq, pq = oracle.quantize(Q8_0, emb), oracle.quantize(Q8_0, proj)
    want_rows = oracle.dequantize(Q8_0, eq, 256).reshape(50, 256)[which]
    assert np.array_equal(out["rows"].reshape(4, 256), want_rows)
    close(out["scores"].reshape(4, 96), oracle.mul_mat(Q8_0, pq, 256, want_rows), 1e-3)
    prog.free()
    f.close()
    n.close()
