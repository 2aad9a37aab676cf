"""GGUF reader / writer against itself and, where the reference's own ggml build is available,
against the reference's reader (vendored gguf.cpp, the one crates/tensorlisp/src/gguf.rs wraps): the
file written here must parse there with the same keys, tensor types, sizes and offsets."""
import numpy as np
import pytest

from tensorlisp_b200 import graph as G
from tensorlisp_b200.gguf import ARRAY, GgufError, GgufFile, GgufWriter, STRING, U32


def write_sample(path, oracle):
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((6, 512)) * 0.02).astype(np.float32)
    out = GgufWriter()
    out.set_str("general.architecture", "llama")
    out.set_program("(define (forward x) (ggml-mul-mat W x))")
    out.set_asset("tokenizer.model", b"\x00\x01binary\xff")
    out.add_tensor("norm", G.F32, [512], np.ones(512, np.float32))
    out.add_tensor("W", G.F32, [512, 6], w)
    out.add_tensor("W.q8", G.Q8_0, [512, 6], oracle.quantize(G.Q8_0, w))
    out.add_tensor("W.q4k", G.Q4_K, [512, 6], oracle.quantize(G.Q4_K, w))
    out.write(str(path))
    return w


def test_round_trip(tmp_path, oracle):
    p = tmp_path / "m.gguf"
    w = write_sample(p, oracle)
    f = GgufFile(str(p))
    assert f.version == 3 and f.alignment == 32 and f.data_offset % 32 == 0
    assert f.program() == "(define (forward x) (ggml-mul-mat W x))"
    assert f.kv["TL_VER"] == (U32, 1) and f.kv["general.architecture"] == (STRING, "llama")
    assert f.assets() == {"tokenizer.model": b"\x00\x01binary\xff"}
    names = [t.name for t in f.tensors]
    assert names == ["norm", "W", "W.q8", "W.q4k"]
    assert all(t.offset % 32 == 0 for t in f.tensors)
    assert np.array_equal(f.tensor_bytes(1).view(np.float32).reshape(6, 512), w)
    assert np.array_equal(f.tensor_bytes(2), oracle.quantize(G.Q8_0, w).reshape(-1))
    assert f.tensors[3].ne == [512, 6] and f.tensors[3].nbytes == 6 * 2 * 144
    f.close()


def test_errors(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(GgufError):
        GgufFile(str(p))
    out = GgufWriter()
    out.set_str("k", "v")
    out.write(str(p))
    f = GgufFile(str(p))
    with pytest.raises(GgufError) as e:
        f.program()
    assert "TL_VER is missing" in str(e.value)
    f.close()
    with pytest.raises(GgufError):
        out.add_tensor("short", G.Q8_0, [64, 2], np.zeros(10, np.uint8))


def test_the_reference_reader_sees_the_same_file(tmp_path, oracle, ref):
    from oracle.bindings import ref_gguf_summary
    p = tmp_path / "m.gguf"
    write_sample(p, oracle)
    text = ref_gguf_summary(ref, str(p))
    if text is None:
        pytest.skip("the reference build in oracle/_ref predates the GGUF hook: rebuild with python oracle/build.py")
    f = GgufFile(str(p))
    lines = text.strip().splitlines()
    assert lines[0] == "version 3 alignment 32 data_offset %d" % f.data_offset
    kv = [l for l in lines if l.startswith("kv ")]
    assert "kv TL_VER u32 1" in kv and "kv TL_TXT string (define (forward x) (ggml-mul-mat W x))" in kv
    assert "kv TL_ASSET.tokenizer.model array 0 9" in kv
    tl = [l for l in lines if l.startswith("tensor ")]
    assert tl == ["tensor %s type %d offset %d size %d" % (t.name, t.ty, t.offset, t.nbytes) for t in f.tensors]
    f.close()
