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


def test_quantize_selection_rules():
    """Which tensors `tl quantize` converts (crates/tensorlisp-cli/src/quantize.rs:54-80,148-191): host logic only."""
    from types import SimpleNamespace as T
    from tensorlisp_b200.gguf import glob_match, skip_reason, weight_uses
    g = G.Graph()
    w = g.weight(G.F32, [256, 8], "w")
    b = g.weight(G.F32, [8], "b")
    e = g.weight(G.F32, [256, 100], "e")
    both = g.weight(G.F32, [256, 8], "both")
    x = g.get_rows(e, g.input(G.I32, [2], "ids"))
    y = g.add(g.mul_mat(g.permute(g.permute(w, 1, 0, 2, 3), 1, 0, 2, 3), x), b)      # w behind two view ops
    y = g.add(y, g.mul_mat(both, x))
    z = g.mul_mat(x, both)            # `both` also as source 1 of a MUL_MAT
    g.output(y)
    g.output(z)
    uses = weight_uses([g])
    assert uses["w"] == [("MUL_MAT", 0)] and uses["e"] == [("GET_ROWS", 0)] and uses["b"] == [("ADD", 1)]
    assert sorted(uses["both"]) == [("MUL_MAT", 0), ("MUL_MAT", 1)]
    info = lambda name, ty, ne: T(name=name, ty=ty, ne=ne, nbytes=0)
    assert skip_reason(info("w", G.F32, [256, 8]), G.Q8_0, uses) is None
    assert skip_reason(info("e", G.F32, [256, 100]), G.Q8_0, uses) is None
    assert skip_reason(info("both", G.F32, [256, 8]), G.Q8_0, uses).startswith("used by MUL_MAT (source 1)")
    assert skip_reason(info("b", G.F32, [8]), G.Q8_0, uses).startswith("used by ADD (source 1)")
    assert skip_reason(info("gone", G.F32, [256, 8]), G.Q8_0, uses) == "not used by the program"
    assert skip_reason(info("w", G.Q8_0, [256, 8]), G.Q8_0, uses) == "already q8_0"
    assert skip_reason(info("w", G.Q4_0, [256, 8]), G.Q8_0, uses) == "already quantized (use --requantize)"
    assert skip_reason(info("w", G.Q4_0, [256, 8]), G.Q8_0, uses, requantize=True) is None
    assert skip_reason(info("w", G.F32, [256, 8]), G.Q8_0, uses, include=["blk.*"]) == "not included"
    assert skip_reason(info("w", G.F32, [256, 8]), G.Q8_0, uses, exclude=["?"]) == "excluded by ?"
    assert skip_reason(info("w", G.I32, [256, 8]), G.Q8_0, None) == "integer tensor"
    assert skip_reason(info("w", G.F32, [256, 2]), G.Q8_0, None) == "fewer than 1024 elements"
    assert skip_reason(info("w", G.F32, [4096]), G.Q8_0, None) == "1-D (use --include-1d)"
    assert skip_reason(info("w", G.F32, [4096]), G.Q8_0, None, include_1d=True) is None
    assert skip_reason(info("w", G.F32, [100, 50]), G.Q4_K, None) == "row length 100 is not a multiple of the q4_K block size 256"
    assert glob_match("blk.*.attn_?", "blk.12.attn_q") and not glob_match("blk.*", "output") and glob_match("*", "")


def test_convert_rules(tmp_path):
    """The decisions of `tl convert` (crates/tensorlisp-cli/src/convert.rs:129-149, 217-224, 271-302), without a GPU: which
    type every tensor is stored as, names, offsets, and the errors raised before any data is read."""
    from helpers import write_safetensors
    from tensorlisp_b200 import graph as G
    from tensorlisp_b200.gguf import GgufError, convert_plan, read_safetensors_header
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, {
        "model.embed.weight": np.zeros((64, 256), np.float32),
        "model.layers.0.attn.weight": np.zeros((256, 256), np.float16),
        "model.layers.0.norm.weight": np.zeros(256, np.float32),
        "model.layers.0.small.weight": np.zeros((2, 256), np.float32),
        "model.layers.0.ragged.weight": ("BF16", np.zeros((40, 100), np.uint16)),
        "model.ids": np.arange(6, dtype=np.int64),
        "model.mask": np.ones((2, 3), np.bool_),
        "model.double": np.zeros((4, 32), np.float64),
    })
    entries, data0 = read_safetensors_header(path)
    assert [e["name"] for e in entries][:2] == ["model.embed.weight", "model.layers.0.attn.weight"] and data0 % 8 == 0
    by = lambda plan: {p["name"]: p for p in plan}
    plan, skipped = convert_plan(entries, "q4_K", no_quant=["*embed*"], strip_prefix=["model."], replace_prefix=["layers.=blk."],
                                 rename=["ids=token_ids"], exclude=["*mask"], offset=["*norm.weight=1"])
    p = by(plan)
    assert skipped == ["model.mask"]
    assert p["model.embed.weight"]["stored"] == G.F16                       # --no-quant: f16 instead
    assert p["model.layers.0.attn.weight"]["stored"] == G.Q4_K
    assert p["model.layers.0.norm.weight"]["stored"] == G.F32 and p["model.layers.0.norm.weight"]["offset"] == 1.0   # 1-D stays f32
    assert p["model.layers.0.small.weight"]["stored"] == G.F16              # fewer than --min-elements values
    assert p["model.layers.0.ragged.weight"]["stored"] == G.F16             # rows of 100 do not fit blocks of 256
    assert p["model.ids"]["stored"] == G.I32 and p["model.ids"]["new_name"] == "token_ids"
    assert p["model.double"]["stored"] == G.F16                             # 128 values: below the minimum
    assert p["model.layers.0.attn.weight"]["new_name"] == "blk.0.attn.weight"
    keep = by(convert_plan(entries, "keep")[0])
    assert keep["model.layers.0.attn.weight"]["stored"] == G.F16 and keep["model.layers.0.ragged.weight"]["stored"] == G.BF16
    assert keep["model.double"]["stored"] == G.F32 and keep["model.mask"]["stored"] == G.I32
    half = by(convert_plan(entries, "bf16")[0])
    assert half["model.embed.weight"]["stored"] == G.BF16 and half["model.layers.0.norm.weight"]["stored"] == G.F32
    mixed = by(convert_plan(entries, "q4_K", types=["*attn*=q8_0", "*norm*=f16"])[0])
    assert mixed["model.layers.0.attn.weight"]["stored"] == G.Q8_0 and mixed["model.layers.0.norm.weight"]["stored"] == G.F16
    with pytest.raises(GgufError):      # a type the rows do not fit is an error before any data is read
        convert_plan(entries, "keep", types=["*ragged*=q4_K"])
    with pytest.raises(GgufError):
        convert_plan(entries, "keep", offset=["model.ids=1"])
    with pytest.raises(GgufError):
        convert_plan(entries, "q9_9")


def test_pack_program_keeps_tensors_and_metadata(tmp_path):
    """`tl pack`: the program and a replaced asset go in, tensors and the other keys stay byte for byte; with no output
    path the file itself is replaced."""
    from tensorlisp_b200 import graph as G
    from tensorlisp_b200.gguf import GgufFile, GgufWriter, pack_program
    path = str(tmp_path / "m.gguf")
    w = np.arange(64, dtype=np.float32).reshape(4, 16)
    out = GgufWriter()
    out.set_str("general.name", "tiny")
    out.set_asset("vocab", b"old")
    out.set_asset("merges", b"m")
    out.add_tensor("w", G.F32, [16, 4], w)
    out.write(path)
    pack_program(path, None, "(define (f x) x)", assets=[("vocab", b"new")])
    f = GgufFile(path)
    assert f.program() == "(define (f x) x)" and f.kv["general.name"][1] == "tiny"
    assert dict(f.assets()) == {"vocab": b"new", "merges": b"m"}
    assert np.array_equal(np.frombuffer(f.tensor_bytes(0), np.float32).reshape(4, 16), w)
    f.close()
    other = str(tmp_path / "n.gguf")
    pack_program(path, other, "(define (g x) x)")
    f = GgufFile(other)
    assert f.program() == "(define (g x) x)" and dict(f.assets())["vocab"] == b"new"
    f.close()
