"""Row / elementwise / gather ops of a decoder graph through compiled programs, against the oracle
and the golden vectors (reference test model: crates/tensorlisp/tests/native.rs, tolerances
:108-153 norms 1e-4, :251-278 rope/argmax 1e-5)."""
import os

import numpy as np
import pytest

from helpers import Model, close
from oracle.bindings import Q8_0
from tensorlisp_b200 import graph as G
from tensorlisp_b200.native import Native, TlbError

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def test_rms_norm_mul_fused_and_unfused(oracle, monkeypatch):
    x, w = GOLD["row_x"], GOLD["row_w"]
    for nofuse in ("", "1"):
        if nofuse:
            monkeypatch.setenv("TL_NATIVE_NOFUSE", nofuse)
        g = G.Graph()
        tx = g.input(G.F32, [384, 6], "x")
        tw = g.weight(G.F32, [384], "w")
        y = g.output(g.mul(g.rms_norm(tx, 1e-5), tw, "y"))
        n = g.output(g.rms_norm(tx, 1e-6, "n"))
        m = Model(g, [w])
        labels = m.program.labels()
        assert len(labels) == (3 if nofuse else 2), labels
        got_y, got_n = m.run(x)
        close(got_y, GOLD["row_rms_mul"], 1e-5)
        close(got_n, GOLD["row_rms"], 1e-5)
        m.close()


def test_norm_second_reader_blocks_fusion():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 64)).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    g = G.Graph()
    tx = g.input(G.F32, [64, 4])
    tw = g.weight(G.F32, [64])
    n = g.rms_norm(tx, 1e-5)
    y = g.output(g.mul(n, tw))
    z = g.output(g.add(n, tx))
    m = Model(g, [w])
    assert len(m.program.labels()) == 3
    gy, gz = m.run(x)
    nn = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    close(gy, nn * w, 1e-5)
    close(gz, nn + x, 1e-5)
    m.close()


def test_narrow_weight_repeats_across_the_row():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 128)).astype(np.float32)
    w = rng.standard_normal(32).astype(np.float32)
    g = G.Graph()
    tx = g.input(G.F32, [128, 3])
    tw = g.weight(G.F32, [32])
    y = g.output(g.mul(g.rms_norm(tx, 1e-5), tw))
    m = Model(g, [w])
    (gy,) = m.run(x)
    nn = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    close(gy, nn * np.tile(w, 4), 1e-5)
    m.close()


@pytest.mark.parametrize("style", ["unary_mul", "glu_split", "glu_packed"])
def test_silu_gate(oracle, style):
    x, u = GOLD["row_x"], GOLD["row_u"]
    g = G.Graph()
    if style == "glu_packed":
        t = g.input(G.F32, [768, 6], "xu")
        y = g.output(g.glu(t, "swiglu"))
        m = Model(g)
        (got,) = m.run(np.concatenate([x, u], axis=1))
    else:
        tx = g.input(G.F32, [384, 6], "x")
        tu = g.input(G.F32, [384, 6], "u")
        y = g.output(g.mul(g.silu(tx), tu) if style == "unary_mul" else g.glu(tx, "swiglu", b=tu))
        m = Model(g)
        if style == "unary_mul":
            assert len(m.program.labels()) == 1  # SiLU and the product are one launch
        (got,) = m.run(x, u)
    close(got, GOLD["row_silu_mul"], 1e-5)
    m.close()


@pytest.mark.parametrize("mode,name,nd,base", [(2, "rope_neox", 128, 500000.0), (0, "rope_normal", 128, 500000.0), (2, "rope_neox_partial", 64, 10000.0)])
def test_rope(mode, name, nd, base):
    x, pos = GOLD["rope_x"], GOLD["rope_pos"]
    g = G.Graph()
    tx = g.input(G.F32, [128, 3, 5], "x")
    tp = g.input(G.I32, [5], "pos")
    y = g.output(g.rope_ext(tx, tp, None, nd, mode, 0, base, 1.0, 0.0, 1.0, 32.0, 1.0))
    m = Model(g)
    (got,) = m.run(x, pos)
    close(got.reshape(5, 3, 128), GOLD[name], 1e-5)
    m.close()


ROPE_VARIANTS = [
    # head, heads, tokens, n_dims, mode, n_ctx_orig, base, freq_scale, ext_factor, attn_factor, beta_fast, beta_slow, freq factors
    (8, 2, 3, 8, 2, 0, 100.0, 0.5, 0.0, 1.0, 32.0, 1.0, False),       # attn:rope 'base 100.0 'scale 0.5 (native.rs:256)
    (8, 2, 3, 8, 0, 0, 100.0, 1.0, 0.0, 1.0, 0.0, 0.0, False),        # ggml-rope-ext ... 8 0 0 100.0 1.0 0.0 1.0 0.0 0.0 (native.rs:257)
    (128, 4, 6, 128, 2, 0, 500000.0, 1.0, 0.0, 1.0, 32.0, 1.0, True),  # per-frequency factors (the scaled-rope models)
    (128, 4, 6, 64, 0, 0, 10000.0, 1.0, 0.0, 1.0, 32.0, 1.0, True),
    (128, 4, 6, 128, 2, 4096, 10000.0, 0.25, 1.0, 1.0, 32.0, 1.0, False),   # YaRN: interpolated and extrapolated angles mixed by a ramp
    (64, 2, 5, 64, 0, 2048, 10000.0, 0.5, 0.7, 1.3, 16.0, 2.0, False),
]


@pytest.mark.parametrize("v", ROPE_VARIANTS, ids=[str(v[:9]) for v in ROPE_VARIANTS])
def test_rope_variants_against_ggml(ref, v):
    """Frequency scale, per-frequency factors and the YaRN ramp against ggml's CPU rope on the same inputs (the reference's
    own test runs the first two at 1e-5, crates/tensorlisp/tests/native.rs:252-275)."""
    hd, heads, tokens, nd, mode, nctx, base, fs, ext, attn, bf, bs, with_ff = v
    rng = np.random.default_rng(hd + nd + mode)
    x = rng.standard_normal((tokens, heads, hd)).astype(np.float32)
    pos = np.array([0, 3, 7, 100, 4095, 8191][:tokens], np.int32)
    ff = (1.0 + 7.0 * rng.random(nd // 2)).astype(np.float32)
    rg = ref.graph(16 << 20, 1)
    rx, rp = rg.tensor(G.F32, [hd, heads, tokens], "x", x), rg.tensor(G.I32, [tokens], "pos", pos)
    rf = rg.tensor(G.F32, [nd // 2], "ff", ff) if with_ff else None
    ry = rg.op("rope_ext", [rx, rp, rf], ints=[nd, mode, nctx], floats=[base, fs, ext, attn, bf, bs])
    rg.compute([ry])
    want = rg.read(ry).reshape(tokens, heads, hd).copy()
    rg.close()
    g = G.Graph()
    tx = g.input(G.F32, [hd, heads, tokens], "x")
    tp = g.input(G.I32, [tokens], "pos")
    tf = g.input(G.F32, [nd // 2], "ff") if with_ff else None
    g.output(g.rope_ext(tx, tp, tf, nd, mode, nctx, base, fs, ext, attn, bf, bs))
    m = Model(g)
    (got,) = m.run(*([x, pos, ff] if with_ff else [x, pos]))
    m.close()
    close(got.reshape(tokens, heads, hd), want, 1e-5)


def test_soft_max_scale_argmax_add():
    x = GOLD["row_x"]
    g = G.Graph()
    tx = g.input(G.F32, [384, 6], "x")
    sm = g.output(g.soft_max_ext(tx, None, 0.25))
    am = g.output(g.argmax(tx))
    sc = g.output(g.scale(tx, 0.5, 0.25))
    ad = g.output(g.add(tx, sc))
    m = Model(g)
    gsm, gam, gsc, gad = m.run(x)
    close(gsm, GOLD["row_softmax"], 1e-5)
    assert np.array_equal(gam, GOLD["row_argmax"])
    close(gsc, x * 0.5 + 0.25, 1e-6)
    close(gad, x + (x * 0.5 + 0.25), 1e-6)
    m.close()


def test_argmax_ties_pick_the_last_index():
    g = G.Graph()
    tx = g.input(G.F32, [40, 3])
    am = g.output(g.argmax(tx))
    m = Model(g)
    (got,) = m.run(GOLD["ties_x"])
    assert np.array_equal(got, GOLD["ties_argmax"])
    m.close()


@pytest.mark.parametrize("n", [100, 16384, 20000, 20001, 262144])
def test_argmax_of_long_rows(n):
    """The rows of the reference's own long-row test (crates/tensorlisp/tests/native.rs:416-436): the same maximum at three
    places of a row, the maximum in the last element, noise. The native CUDA executor and ggml's CPU backend keep the
    LAST of equal maxima (crates/kernels/src/cuda/native/core.cu:456-460). 20001 makes every second row start off a 16-byte
    boundary."""
    rng = np.random.default_rng(n)
    x = rng.standard_normal((3, n)).astype(np.float32)
    for j in (n // 3, n // 2 + 1, n - 1):
        x[0, j] = 5.0
    x[1, n - 1] = 9.0
    g = G.Graph()
    tx = g.input(G.F32, [n, 3])
    g.output(g.argmax(tx))
    m = Model(g)
    (got,) = m.run(x)
    m.close()
    want = np.array([n - 1 - int(np.argmax(x[r, ::-1])) for r in range(3)], np.int32)
    assert np.array_equal(np.asarray(got).reshape(-1), want)


def test_masked_soft_max():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 5, 64)).astype(np.float32)       # [heads, rows, n]
    mask = np.where(rng.random((5, 64)) < 0.3, -np.inf, 0).astype(np.float16)
    mask[:, 0] = 0
    g = G.Graph()
    tx = g.input(G.F32, [64, 5, 2])
    tm = g.input(G.F16, [64, 5])
    y = g.output(g.soft_max_ext(tx, tm, 0.5))
    m = Model(g)
    (got,) = m.run(x, mask)
    z = x.astype(np.float64) * 0.5 + mask.astype(np.float64)
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    close(got, e / e.sum(axis=-1, keepdims=True), 1e-5)
    m.close()


def test_get_rows_q8_0_table(oracle):
    tab = oracle.quantize(Q8_0, GOLD["emb_table"])
    g = G.Graph()
    tt = g.weight(G.Q8_0, [256, 50], "emb")
    ti = g.input(G.I32, [5], "ids")
    y = g.output(g.get_rows(tt, ti))
    m = Model(g, [tab])
    (got,) = m.run(GOLD["emb_ids"])
    assert np.array_equal(got, GOLD["emb_rows"])
    m.close()


def test_casts_and_permuted_copy():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 4, 8)).astype(np.float32)
    g = G.Graph()
    tx = g.input(G.F32, [8, 4, 3])
    h = g.cast(tx, G.F16)
    back = g.output(g.cast(h, G.F32))
    pc = g.output(g.cont(g.permute(tx, 0, 2, 1, 3)))
    m = Model(g)
    gb, gp = m.run(x)
    assert np.array_equal(gb, x.astype(np.float16).astype(np.float32))
    assert np.array_equal(gp, x.transpose(1, 0, 2))
    m.close()


def test_state_persists_and_sessions_are_separate():
    """SET_ROWS into a state tensor survives runs; reset_state / new_state_block / fork_block behave
    like the reference's sessions (crates/tensorlisp/tests/native.rs:436-468)."""
    g = G.Graph()
    cache = g.state(G.F16, [16, 8], "cache")
    rows = g.input(G.F32, [16, 2], "rows")
    ids = g.input(G.I64, [2], "ids")
    wr = g.set_rows(cache, rows, ids)
    out = g.output(g.cast(wr, G.F32))
    m = Model(g, state_bytes=[16 * 8 * 2])
    r1 = np.arange(32, dtype=np.float32).reshape(2, 16)
    (a,) = m.run(r1, np.array([1, 5], np.int64))
    assert np.array_equal(a[1], r1[0]) and np.array_equal(a[5], r1[1]) and not a[0].any()
    (b,) = m.run(r1 + 100, np.array([0, 7], np.int64))
    assert np.array_equal(b[1], r1[0]) and np.array_equal(b[0], r1[0] + 100)   # first write still there
    other = m.native.new_state_block()
    (c,) = m.run(r1, np.array([2, 3], np.int64), state=other)
    assert not c[1].any() and np.array_equal(c[2], r1[0])                        # a fresh session is zeroed
    fork = m.native.fork_block(other)
    (d,) = m.run(r1 + 1, np.array([4, 6], np.int64), state=fork)
    assert np.array_equal(d[2], r1[0]) and np.array_equal(d[4], r1[0] + 1)
    m.native.reset_state()
    (e,) = m.run(r1, np.array([-1, 7], np.int64))
    assert not e[:7].any() and np.array_equal(e[7], r1[1])                       # negative row ids are skipped
    m.close()


def test_unsupported_op_is_reported_by_name():
    """crates/tensorlisp/tests/native.rs:240-249: CUMSUM + "not implemented"."""
    g = G.Graph()
    tx = g.input(G.F32, [8, 2])
    a = g.cumsum(tx, "c1")
    b = g.cumsum(a, "c2")
    y = g.output(g.add(b, tx))
    with pytest.raises(TlbError) as e:
        Model(g)
    msg = str(e.value)
    assert msg.startswith("native CUDA: not implemented: CUMSUM x2 (e.g. c1:"), msg
    assert e.value.kind == "Unsupported"


def test_input_size_is_checked():
    g = G.Graph()
    tx = g.input(G.F32, [8, 2])
    y = g.output(g.scale(tx, 2.0))
    m = Model(g)
    with pytest.raises(TlbError) as e:
        m.program.set_input(0, np.zeros(15, np.float32))
    assert str(e.value) == "input 0 takes 64 bytes, got 60"
    with pytest.raises(TlbError):
        m.program.set_input(3, np.zeros(16, np.float32))
    m.close()


def test_empty_tensors_launch_nothing():
    g = G.Graph()
    tx = g.input(G.F32, [8, 0])
    y = g.output(g.scale(tx, 2.0))
    m = Model(g)
    assert m.program.dispatch_count() == 0
    m.program.run()
    m.close()


def test_device_name():
    from tensorlisp_b200.native import Native
    n = Native(0)
    assert n.device_name().startswith("native ")
    n.close()


def test_copy_blocks_copies_pairs():
    """The reference's own check (crates/kernels/tests/paged_attn_cuda.rs:269-299): pairs (0 -> 4) and (2 -> 5) of a
    6-page pool, in the K pool and the V pool of one state block; other pages keep their bytes; bad pairs are refused."""
    from tensorlisp_b200._lib import TlbError
    nb, n = 6, 40 * 4            # pages of 160 f32 = 640 bytes
    kc = np.arange(nb * n, dtype=np.float32)
    vc = -kc
    native = Native.load([])
    native.alloc_states([kc.nbytes, vc.nbytes])
    ko, vo = native.state_offsets
    native.state.write(ko, kc)
    native.state.write(vo, vc)
    native.state.copy_blocks(ko, vo, nb, n * 4, [(0, 4), (2, 5)])
    k2 = native.state.read(ko, kc.nbytes).view(np.float32)
    v2 = native.state.read(vo, vc.nbytes).view(np.float32)
    for src, dst in ((0, 4), (2, 5)):
        assert np.array_equal(k2[dst * n:(dst + 1) * n], kc[src * n:(src + 1) * n])
        assert np.array_equal(v2[dst * n:(dst + 1) * n], vc[src * n:(src + 1) * n])
    for blk in (0, 1, 2, 3):
        assert np.array_equal(k2[blk * n:(blk + 1) * n], kc[blk * n:(blk + 1) * n]), "untouched block changed"
        assert np.array_equal(v2[blk * n:(blk + 1) * n], vc[blk * n:(blk + 1) * n])
    for bad in ([(0, 6)], [(0, 4), (4, 5)], [(1, 3), (2, 3)], [(-1, 2)]):
        with pytest.raises(TlbError):
            native.state.copy_blocks(ko, vo, nb, n * 4, bad)
    native.close()


def test_entry_cache_compiles_per_shape_and_converts_i32_inputs():
    """The caller side of the boundary (Inner::run_native, crates/tensorlisp/src/model.rs:1038-1093): an entry is compiled
    for the shapes of its inputs when they are first seen and replayed afterwards; an i32 input arrives as whole-number f32
    values."""
    from tensorlisp_b200.native import EntryCache, Native
    rng = np.random.default_rng(31)
    table = rng.standard_normal((20, 64)).astype(np.float32)
    built = []

    def build(name, shapes):
        built.append(shapes)
        g = G.Graph()
        w = g.weight(G.F32, [64, 20], "table")
        ids = g.input(G.I32, [shapes[0][0]], "ids")
        x = g.input(G.F32, [64, shapes[1][0]], "x")
        g.output(g.get_rows(w, ids, "rows"))
        g.output(g.mul_mat(w, x, "scores"))
        return g

    n = Native.load([table])
    n.alloc_states([])
    cache = EntryCache(n, build)
    for n_ids, n_x in ((3, 2), (5, 2), (3, 2)):
        ids = rng.integers(0, 20, n_ids).astype(np.float32)          # whole numbers as f32, as the caller passes them
        x = rng.standard_normal((n_x, 64)).astype(np.float32)
        out = dict(cache.run("lookup", [ids, x]))
        assert np.array_equal(out["rows"].reshape(n_ids, 64), table[ids.astype(int)])
        close(out["scores"].reshape(n_x, 20), x @ table.T, 1e-5)
    assert built == [((3,), (2, 64)), ((5,), (2, 64))]               # the third call reused the first program
    with pytest.raises(ValueError):
        cache.run("lookup", [np.array([0.5, 1, 2], np.float32), np.zeros((2, 64), np.float32)])
    cache.free()
    n.close()
