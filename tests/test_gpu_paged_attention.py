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
    g.paged_cache_write(g.cast(tk, G.F16), g.cast(tv, G.F16), kc, vc, ts, bs, kvh)
    pa = g.paged_attention(g.cast(tq, G.F16), kc, vc, tt, tl, bs, max_ctx, scale, kvh)
    out = g.output(g.cast(pa, G.F32))
    m = Model(g, state_bytes=[pool_elems * 2, pool_elems * 2])
    (got,) = m.run(q.astype(np.float32), key.astype(np.float32), val.astype(np.float32), tables, ctxs,
                   slots.view(np.int32))
    want16, want32 = oracle.attention_decode(q, ks, vs, kvh, scale)
    m.close()
    return got.reshape(seqs, heads, hs), want32


@pytest.mark.parametrize("hs,kvh,heads,bs", [(64, 1, 4, 16), (128, 2, 8, 8), (256, 1, 2, 16), (128, 8, 32, 16), (128, 2, 2, 32), (64, 1, 20, 16)])
def test_paged_matches_dense(oracle, hs, kvh, heads, bs):
    got, want = paged_case(oracle, 4, heads, kvh, hs, bs, [1, 17, 64, 150], seed=hs + bs)
    close(got, want, 1e-3)


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
