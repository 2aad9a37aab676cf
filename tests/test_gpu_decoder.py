"""End-to-end parity of the SwiGLU FFN block (BASELINE config 2) and of a whole decode step of a
Llama-shaped decoder (BASELINE config 4 at reduced depth / vocabulary, same per-layer geometry rules)
against the oracle. Bars (BASELINE north_star): mul_mat chains 1e-3 of max|want|; end-to-end logits
within 1e-2 absolute with identical top-1."""
import numpy as np
import pytest

from helpers import Model, close, make_decoder_weights, oracle_decoder_step
from oracle.bindings import Q4_K
from tensorlisp_b200 import graph as G
from tensorlisp_b200.programs import DecoderConfig, decoder_step, decoder_weights, swiglu_ffn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T", [1, 32])
def test_ffn_block_config2(oracle, T):
    """RMSNorm(eps 1e-5, w ~ N(1, 0.1)) -> gate/up 4096->14336 Q4_K -> SiLU(gate)*up -> down 14336->4096."""
    d, f = 4096, 14336
    rng = np.random.default_rng(2)
    wn = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    from tensorlisp_b200.native import Native, quantize_rows
    n = Native(0)
    mats = []
    for rows, cols in ((f, d), (f, d), (d, f)):
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
        mats.append(quantize_rows(n, Q4_K, w))   # bit-exact with the oracle (tests/test_gpu_quantize.py)
    n.close()
    x = rng.standard_normal((T, d)).astype(np.float32)
    g = G.Graph()
    tn = g.weight(G.F32, [d], "norm")
    tg = g.weight(G.Q4_K, [d, f], "gate")
    tu = g.weight(G.Q4_K, [d, f], "up")
    td = g.weight(G.Q4_K, [f, d], "down")
    tx = g.input(G.F32, [d, T], "x")
    y = g.output(swiglu_ffn(g, tx, tn, tg, tu, td, 1e-5))
    m = Model(g, [wn] + mats)
    (got,) = m.run(x)
    h = oracle.rms_norm(x, 1e-5, wn)
    a = oracle.mul_mat(Q4_K, mats[0], d, h)
    b = oracle.mul_mat(Q4_K, mats[1], d, h)
    want = oracle.mul_mat(Q4_K, mats[2], f, oracle.silu_mul(a, b))
    close(got, want, 1e-3)
    m.close()


def test_decode_step_logits_and_top1(oracle):
    cfg = DecoderConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ffn=1024, vocab=1024)
    B, max_ctx, bs = 3, 64, cfg.block_size
    rng = np.random.default_rng(5)
    ctx_before = np.array([0, 17, 40], np.int32)          # tokens already cached per sequence
    pos = ctx_before.copy()
    lens = ctx_before + 1
    ids = rng.integers(0, cfg.vocab, B).astype(np.int32)
    max_blocks = max_ctx // bs
    pool_blocks = B * max_blocks
    dg = decoder_step(cfg, B, max_ctx, pool_blocks)
    weights = make_decoder_weights(oracle, dg.weights, seed=9)
    tables = rng.permutation(pool_blocks).astype(np.int32).reshape(B, max_blocks)
    slots = np.array([tables[b, pos[b] // bs] * bs + pos[b] % bs for b in range(B)], np.int64)

    m = Model(dg.graph, weights, dg.state_bytes)
    # pre-fill the pools with the cached tokens: layout [block][kv_head][slot][hd]
    kvh, hd = cfg.n_kv_heads, cfg.head_dim
    ks = [[np.zeros((lens[b], kvh, hd), np.float16) for b in range(B)] for _ in range(cfg.n_layers)]
    vs = [[np.zeros((lens[b], kvh, hd), np.float16) for b in range(B)] for _ in range(cfg.n_layers)]
    for l in range(cfg.n_layers):
        kp = np.zeros((pool_blocks, kvh, bs, hd), np.float16)
        vp = np.zeros((pool_blocks, kvh, bs, hd), np.float16)
        for b in range(B):
            ks[l][b][:ctx_before[b]] = rng.standard_normal((ctx_before[b], kvh, hd)).astype(np.float16)
            vs[l][b][:ctx_before[b]] = rng.standard_normal((ctx_before[b], kvh, hd)).astype(np.float16)
            for t in range(ctx_before[b]):
                kp[tables[b, t // bs], :, t % bs] = ks[l][b][t]
                vp[tables[b, t // bs], :, t % bs] = vs[l][b][t]
        m.native.state.write(m.native.state_offsets[2 * l], kp)
        m.native.state.write(m.native.state_offsets[2 * l + 1], vp)
    logits, token = m.run(ids, pos, tables, lens, slots.view(np.int32))
    want = oracle_decoder_step(oracle, cfg, dg.weights, weights, ids, pos, ks, vs)
    assert np.abs(logits - want).max() <= 1e-2
    assert np.array_equal(logits.argmax(axis=1), want.argmax(axis=1))
    assert np.array_equal(token.astype(np.int64), want.argmax(axis=1))
    m.close()
