"""Paged cache write + paged-attention decode through compiled programs (the CUSTOM nodes of
scheme/core.ss:222-271) against the oracle's closed-form f32 attention over the same f16 K/V
(reference tests: crates/tensorlisp/tests/native.rs:352-410 paged vs dense 4e-3;
crates/kernels/tests/paged_attn_cuda.rs:39-56 f16 tolerance 3e-3). Bar here: 1e-3 of max|want|
plus half an ulp of the f16 output."""
import numpy as np
import pytest

from helpers import Model, close
from tensorlisp_b200 import graph as G

pytestmark = pytest.mark.gpu


def paged_case(oracle, seqs, heads, kvh, hs, bs, ctxs, seed=0, shuffle=True, skip_some=False):
    rng = np.random.default_rng(seed)
    ctxs = np.asarray(ctxs, np.int32)
    max_ctx = int(max(ctxs.max(), 1))
    max_blocks = (max_ctx + bs - 1) // bs
    n_blocks = int(sum((c + bs - 1) // bs for c in ctxs)) + 1
    perm = rng.permutation(n_blocks) if shuffle else np.arange(n_blocks)[::-1].copy()
    tables = np.zeros((seqs, max_blocks), np.int32)
    nxt = 0
    for s, c in enumerate(ctxs):
        nb = (c + bs - 1) // bs
        tables[s, :nb] = perm[nxt:nxt + nb]
        nxt += nb
    scale = 1.0 / np.sqrt(hs)
    q = rng.standard_normal((seqs, heads, hs)).astype(np.float16)
    ks = [rng.standard_normal((c, kvh, hs)).astype(np.float16) for c in ctxs]
    vs = [rng.standard_normal((c, kvh, hs)).astype(np.float16) for c in ctxs]
    # all tokens of all sequences are written in one cache-write node
    tokens = int(ctxs.sum())
    key = np.concatenate(ks).reshape(tokens, kvh * hs) if tokens else np.zeros((0, kvh * hs), np.float16)
    val = np.concatenate(vs).reshape(tokens, kvh * hs) if tokens else np.zeros((0, kvh * hs), np.float16)
    slots = np.zeros(tokens, np.int64)
    i = 0
    for s, c in enumerate(ctxs):
        for t in range(c):
            slots[i] = tables[s, t // bs] * bs + t % bs
            i += 1
    extra = 0
    if skip_some and tokens:
        # extra tokens with negative slots must be skipped
        extra = 3
        key = np.concatenate([key, np.full((extra, kvh * hs), 99, np.float16)])
        val = np.concatenate([val, np.full((extra, kvh * hs), 99, np.float16)])
        slots = np.concatenate([slots, np.full(extra, -1, np.int64)])

    pool_elems = n_blocks * kvh * bs * hs
    g = G.Graph()
    kc = g.state(G.F16, [pool_elems], "pk")
    vc = g.state(G.F16, [pool_elems], "pv")
    tq = g.input(G.F32, [hs, heads, seqs], "q")
    tk = g.input(G.F32, [hs * kvh, tokens + extra], "k")
    tv = g.input(G.F32, [hs * kvh, tokens + extra], "v")
    tt = g.input(G.I32, [max_blocks, seqs], "tables")
    tl = g.input(G.I32, [seqs], "lens")
    ts = g.input(G.I32, [2 * (tokens + extra)], "slots")
    # the constructors take the block sizes the reference's scheme layer allows (8, 16, 32); the executor itself
    # takes any power of two, reached here by rewriting the block-size byte of the nodes' userdata
    gbs = bs if bs in (8, 16, 32) else 8
    cw = g.paged_cache_write(g.cast(tk, G.F16), g.cast(tv, G.F16), kc, vc, ts, gbs, kvh)
    pa = g.paged_attention(g.cast(tq, G.F16), kc, vc, tt, tl, gbs, max_ctx, scale, kvh)
    for node in (cw, pa):
        g.tensors[node].op_params[4] = (g.tensors[node].op_params[4] & ~0xff00) | (bs << 8)
    out = g.output(g.cast(pa, G.F32))
    m = Model(g, state_bytes=[pool_elems * 2, pool_elems * 2])
    (got,) = m.run(q.astype(np.float32), key.astype(np.float32), val.astype(np.float32), tables, ctxs,
                   slots.view(np.int32))
    want16, want32 = oracle.attention_decode(q, ks, vs, kvh, scale)
    m.close()
    return got.reshape(seqs, heads, hs), want32


@pytest.mark.parametrize("hs,kvh,heads,bs", [(64, 1, 4, 16), (128, 2, 8, 8), (256, 1, 2, 16), (128, 8, 32, 16), (128, 2, 2, 32), (64, 1, 20, 16),
                                             # the other head sizes of the reference's list (paged_attn.rs:24), (512, 1, 32) being the
                                             # case of its own test (native.rs:355)
                                             (512, 1, 4, 32), (80, 2, 4, 16), (96, 1, 3, 8), (112, 1, 2, 16), (192, 2, 4, 32)])
def test_paged_matches_dense(oracle, hs, kvh, heads, bs):
    got, want = paged_case(oracle, 4, heads, kvh, hs, bs, [1, 17, 64, 150], seed=hs + bs)
    close(got, want, 1e-3)


@pytest.mark.parametrize("bs", [1, 4, 64])
def test_block_sizes_outside_the_scheme_layer(oracle, bs):
    """Pages of fewer than 8 tokens take the copy path with a table lookup per row; pages longer than a tile span tiles."""
    got, want = paged_case(oracle, 3, 8, 2, 128, bs, [5, 70, 131], seed=bs)
    close(got, want, 1e-3)


def test_head_size_512_ragged_lengths(oracle):
    """The kernel for the head sizes outside 64 / 128 / 256 takes a whole context per CTA: an empty sequence, lengths
    that leave some warps without a token, a context of a thousand tokens, grouped heads."""
    got, want = paged_case(oracle, 5, 4, 2, 512, 16, [0, 1, 3, 1025, 700], seed=5)
    close(got, want, 1e-3)


def test_gather_returns_what_the_cache_write_stored():
    """gather_kv_cache of the reference's paged-attention module (crates/kernels/src/cuda/paged_attn.rs:450-509; its own
    check: crates/kernels/tests/paged_attn_cuda.rs:140-170): tokens written through the cache-write node into shuffled
    pages come back, sequence after sequence, exactly as they went in. Lengths and block numbers outside the tables or
    the pool are refused before anything is launched."""
    from tensorlisp_b200._lib import TlbError
    rng = np.random.default_rng(21)
    kvh, hs, bs, lens = 2, 128, 16, np.array([37, 0, 16, 5], np.int32)
    max_blocks = 3
    n_blocks = 9
    perm = rng.permutation(n_blocks)
    tables = np.zeros((len(lens), max_blocks), np.int32)
    nxt = 0
    for s, c in enumerate(lens):
        nb = (c + bs - 1) // bs
        tables[s, :nb] = perm[nxt:nxt + nb]
        nxt += nb
    tokens = int(lens.sum())
    key = rng.standard_normal((tokens, kvh * hs)).astype(np.float16)
    val = rng.standard_normal((tokens, kvh * hs)).astype(np.float16)
    slots = np.concatenate([tables[s, np.arange(c) // bs] * bs + np.arange(c) % bs for s, c in enumerate(lens)]).astype(np.int64)
    pool_elems = n_blocks * kvh * bs * hs
    g = G.Graph()
    kc = g.state(G.F16, [pool_elems], "pk")
    vc = g.state(G.F16, [pool_elems], "pv")
    tk = g.input(G.F32, [hs * kvh, tokens], "k")
    tv = g.input(G.F32, [hs * kvh, tokens], "v")
    ts = g.input(G.I32, [2 * tokens], "slots")
    g.output(g.cast(g.paged_cache_write(g.cast(tk, G.F16), g.cast(tv, G.F16), kc, vc, ts, bs, kvh), G.F32))
    m = Model(g, state_bytes=[pool_elems * 2, pool_elems * 2])
    m.run(key.astype(np.float32), val.astype(np.float32), slots.view(np.int32))
    ko, vo = m.native.state_offsets
    k, v = m.native.state.gather_kv(ko, vo, n_blocks, kvh, hs, bs, tables, lens)
    assert np.array_equal(k.reshape(tokens, kvh * hs), key) and np.array_equal(v.reshape(tokens, kvh * hs), val)
    for bad_tables, bad_lens in ((tables, np.array([49, 0, 16, 5], np.int32)), (np.where(tables == perm[0], n_blocks, tables), lens),
                                 (np.where(tables == perm[0], -1, tables), lens), (tables, np.array([37, -1, 16, 5], np.int32))):
        with pytest.raises(TlbError):
            m.native.state.gather_kv(ko, vo, n_blocks, kvh, hs, bs, bad_tables, bad_lens)
    m.close()


def test_reversed_tables_and_negative_slots(oracle):
    got, want = paged_case(oracle, 3, 8, 2, 128, 16, [33, 5, 100], seed=1, shuffle=False, skip_some=True)
    close(got, want, 1e-3)


def test_split_context_and_ragged_lengths(oracle):
    """Long contexts are split into chunks merged by the reduce kernel; lengths are ragged, one
    sequence is empty, one is exactly a chunk boundary."""
    got, want = paged_case(oracle, 6, 8, 2, 128, 16, [0, 1, 512, 513, 1000, 777], seed=2)
    close(got, want, 1e-3)
    assert not got[0].any()


def test_config3_shape_reduced(oracle):
    """benchmark config 3 geometry (32 q heads, 8 kv heads, hd 128, 16-token pages, permuted pool) at
    8 sequences with contexts drawn from U[128, 8192]."""
    ctxs = np.random.default_rng(3).integers(128, 8193, 8)
    got, want = paged_case(oracle, 8, 32, 8, 128, 16, ctxs, seed=3)
    close(got, want, 1e-3)


def test_config3_full_size(oracle):
    """benchmark config 3 as it is stated: 64 sequences, contexts drawn from U[128, 8192] (seeded, about 266 k cached
    tokens, 1.1 GB of f16 K/V in 16-token pages behind a permuted block table), 32 query heads over 8 KV heads of 128."""
    ctxs = np.random.default_rng(3).integers(128, 8193, 64)
    got, want = paged_case(oracle, 64, 32, 8, 128, 16, ctxs, seed=33)
    close(got, want, 1e-3)


def _bad_index_model(seqs=2, heads=4, kvh=2, hs=64, bs=16, max_ctx=48, n_blocks=6):
    """A cache write and a paged attention over pools of `n_blocks` pages; returns the model and its shapes."""
    max_blocks = (max_ctx + bs - 1) // bs
    tokens = 4
    pool_elems = n_blocks * kvh * bs * hs
    g = G.Graph()
    kc = g.state(G.F16, [pool_elems], "pk")
    vc = g.state(G.F16, [pool_elems], "pv")
    tq = g.input(G.F32, [hs, heads, seqs], "q")
    tk = g.input(G.F32, [hs * kvh, tokens], "k")
    tv = g.input(G.F32, [hs * kvh, tokens], "v")
    tt = g.input(G.I32, [max_blocks, seqs], "tables")
    tl = g.input(G.I32, [seqs], "lens")
    ts = g.input(G.I32, [2 * tokens], "slots")
    g.paged_cache_write(g.cast(tk, G.F16), g.cast(tv, G.F16), kc, vc, ts, bs, kvh)
    g.output(g.cast(g.paged_attention(g.cast(tq, G.F16), kc, vc, tt, tl, bs, max_ctx, 0.125, kvh), G.F32))
    m = Model(g, state_bytes=[pool_elems * 2, pool_elems * 2])
    rng = np.random.default_rng(5)
    inputs = dict(q=rng.standard_normal((seqs, heads, hs)).astype(np.float32),
                  k=rng.standard_normal((tokens, kvh * hs)).astype(np.float32),
                  v=rng.standard_normal((tokens, kvh * hs)).astype(np.float32),
                  tables=np.arange(seqs * max_blocks, dtype=np.int32).reshape(seqs, max_blocks) % n_blocks,
                  lens=np.full(seqs, max_ctx, np.int32), slots=np.arange(tokens, dtype=np.int64))
    return m, inputs


def _run_bad(m, inputs):
    return m.run(inputs["q"], inputs["k"], inputs["v"], inputs["tables"], inputs["lens"], inputs["slots"].view(np.int32))


@pytest.mark.parametrize("what", ["length beyond the tables", "negative length", "block id beyond the pool", "negative block id",
                                  "slot beyond the pool"])
def test_indices_outside_the_tables_or_pools_are_skipped_and_reported(what):
    """A context length, block id or cache slot that points outside the block tables or the pools never becomes an
    address: the kernel skips it and sets the program's error word, the run returns Execution with a message that
    names the cause, and the same program runs cleanly right afterwards with good inputs."""
    from tensorlisp_b200._lib import TLB_EXECUTION, TlbError
    m, good = _bad_index_model()
    (clean,) = _run_bad(m, good)
    bad = {k: v.copy() for k, v in good.items()}
    if what == "length beyond the tables":
        bad["lens"][1] = 48 + 1000
    elif what == "negative length":
        bad["lens"][0] = -7
    elif what == "block id beyond the pool":
        bad["tables"][1, 2] = 6          # pools hold pages 0..5
    elif what == "negative block id":
        bad["tables"][0, 0] = -3
    else:
        bad["slots"][2] = 6 * 16         # first slot past the last page
    with pytest.raises(TlbError) as e:
        _run_bad(m, bad)
    assert e.value.status == TLB_EXECUTION and "out of range" in str(e.value)
    (again,) = _run_bad(m, good)
    assert np.array_equal(again, clean)
    m.close()


def test_cache_write_with_block_size_zero_is_refused():
    from tensorlisp_b200._lib import TlbError
    g = G.Graph()
    kc = g.state(G.F16, [4096], "pk")
    vc = g.state(G.F16, [4096], "pv")
    tk = g.input(G.F32, [128, 2], "k")
    tv = g.input(G.F32, [128, 2], "v")
    ts = g.input(G.I32, [4], "slots")
    node = g.paged_cache_write(g.cast(tk, G.F16), g.cast(tv, G.F16), kc, vc, ts, 8, 2)
    g.tensors[node].op_params[4] &= ~0xff00      # the host mirror refuses a block size of 0 itself: clear the bits behind it
    g.output(node)
    with pytest.raises(TlbError) as e:
        Model(g, state_bytes=[8192, 8192])
    assert "block size" in str(e.value)
