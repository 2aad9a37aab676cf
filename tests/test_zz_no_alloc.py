"""tlb_paged_attention_static: paged-attention decode for callers that may not allocate device memory
(a decode loop that keeps the allocator off its latency path, a host held to a fixed reservation).
Its scratch is a fixed array inside the library instead of arena memory; inputs and outputs are the
caller's. The results must be those of the same attention run through a compiled program, on two
calls in a row (the array keeps the first call's partial sums when the second one starts).

This file is collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C
import os

import numpy as np
import pytest

from helpers import Model
from tensorlisp_b200 import graph as G
from tensorlisp_b200._lib import TLB_INVALID, check, lib

pytestmark = pytest.mark.gpu


def test_static_scratch_attention_matches_the_program_path():
    seqs, heads, kvh, hs, bs = 5, 8, 2, 128, 16
    ctxs = np.array([700, 1, 1536, 333, 64], np.int32)      # long enough for several context chunks
    rng = np.random.default_rng(11)
    max_ctx = int(ctxs.max())
    max_blocks = (max_ctx + bs - 1) // bs
    n_blocks = int(sum((c + bs - 1) // bs for c in ctxs))
    perm = rng.permutation(n_blocks)
    tables = np.zeros((seqs, max_blocks), np.int32)
    nxt = 0
    for s, c in enumerate(ctxs):
        nb = (c + bs - 1) // bs
        tables[s, :nb] = perm[nxt:nxt + nb]
        nxt += nb
    tokens = int(ctxs.sum())
    key = rng.standard_normal((tokens, kvh * hs)).astype(np.float32)
    val = rng.standard_normal((tokens, kvh * hs)).astype(np.float32)
    slots = np.concatenate([tables[s, np.arange(c) // bs].astype(np.int64) * bs + np.arange(c) % bs for s, c in enumerate(ctxs)])
    scale = 1.0 / np.sqrt(hs)
    pool_elems = n_blocks * kvh * bs * hs

    # the existing path: cache write + paged attention as nodes of a compiled program
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
    pa = g.output(g.paged_attention(g.cast(tq, G.F16), kc, vc, tt, tl, bs, max_ctx, scale, kvh))
    m = Model(g, state_bytes=[pool_elems * 2, pool_elems * 2])
    L = lib()
    n = m.native
    q_dev, t_dev, l_dev, o_dev = (n._zeroed(seqs * heads * hs * 2), n._zeroed(tables.nbytes), n._zeroed(ctxs.nbytes),
                                  n._zeroed(seqs * heads * hs * 2))
    t_dev.write(0, tables)
    l_dev.write(0, ctxs)
    kptr = n.state.device_ptr + n.state_offsets[0]
    vptr = n.state.device_ptr + n.state_offsets[1]

    for call in range(2):   # two calls in a row, with different queries
        q = rng.standard_normal((seqs, heads, hs)).astype(np.float32)
        (want,) = m.run(q, key, val, tables, ctxs, slots.view(np.int32))      # fills the pools, then attends
        q_dev.write(0, q.astype(np.float16))
        check(L.tlb_paged_attention_static(n.dev, C.c_void_p(q_dev.device_ptr), C.c_void_p(kptr), C.c_void_p(vptr),
                                           C.c_void_p(t_dev.device_ptr), C.c_void_p(l_dev.device_ptr),
                                           C.c_void_p(o_dev.device_ptr), seqs, heads, kvh, hs, bs, max_blocks, max_ctx, scale))
        got = o_dev.read(0, seqs * heads * hs * 2).view(np.float16).reshape(seqs, heads, hs)
        want = want.reshape(seqs, heads, hs)
        # same kernels, same chunking: the tolerance of the attention tests (1e-3 of max|want|) is met with equality
        err = np.abs(got.astype(np.float32) - want.astype(np.float32)).max()
        assert err <= 1e-3 * np.abs(want.astype(np.float32)).max(), (call, err)
        assert np.array_equal(got, want), call

    # a shape whose partial sums do not fit the built-in array is refused, not truncated (the chunk
    # length is forced down to 64 tokens: the planner's own choice splits a context only as far as it
    # takes to fill the GPU, which keeps the partial sums of any realistic shape far below the limit)
    os.environ["TLB_PA_CHUNK"] = "64"
    st = L.tlb_paged_attention_static(n.dev, C.c_void_p(q_dev.device_ptr), C.c_void_p(kptr), C.c_void_p(vptr),
                                      C.c_void_p(t_dev.device_ptr), C.c_void_p(l_dev.device_ptr), C.c_void_p(o_dev.device_ptr),
                                      4096, 64, 8, 128, 16, 4096, 65535, scale)
    del os.environ["TLB_PA_CHUNK"]
    assert st == TLB_INVALID and b"built-in scratch holds" in L.tlb_last_error()

    # a context length beyond the table row is cut on the device and reported, not followed past the row; the
    # next call with the true lengths gives the same bytes as before
    from tensorlisp_b200._lib import TLB_EXECUTION
    bad = ctxs.copy()
    bad[2] = max_ctx + 5000
    l_dev.write(0, bad)
    args = (n.dev, C.c_void_p(q_dev.device_ptr), C.c_void_p(kptr), C.c_void_p(vptr), C.c_void_p(t_dev.device_ptr),
            C.c_void_p(l_dev.device_ptr), C.c_void_p(o_dev.device_ptr), seqs, heads, kvh, hs, bs, max_blocks, max_ctx, scale)
    assert L.tlb_paged_attention_static(*args) == TLB_EXECUTION and b"out of range" in L.tlb_last_error()
    l_dev.write(0, ctxs)
    check(L.tlb_paged_attention_static(*args))
    assert np.array_equal(o_dev.read(0, seqs * heads * hs * 2).view(np.float16).reshape(seqs, heads, hs), got)
    for b in (q_dev, t_dev, l_dev, o_dev):
        b.free()
    m.close()
