"""The greedy decode loop over the paged pool (tensorlisp_b200.programs.DecodeLoop): N steps of a batch, token ids fed
back on the device, positions / lengths / slots advanced by the host.

 * batched == sequential (the reference's own check, crates/tensorlisp/tests/native_concurrency.rs:174-196): the batch
   of three sequences, started at different context lengths, chooses the same tokens over N steps as three
   single-sequence loops over the same pools.
 * against the oracle: the oracle decodes each sequence on its own, step by step, fed the tokens the GPU chose
   (so one flipped argmax does not send the two runs down different paths); its logits are compared at every step.
"""
import numpy as np
import pytest

from helpers import NoisyOracle, make_decoder_weights, oracle_decoder_step
from tensorlisp_b200.native import Native
from tensorlisp_b200.programs import DecodeLoop, DecoderConfig, decoder_weights

pytestmark = pytest.mark.gpu


def fill_pools(native, cfg, tables, ks, vs, cached):
    bs, kvh, hd = cfg.block_size, cfg.n_kv_heads, cfg.head_dim
    pool_blocks = int(tables.max()) + 1
    for l in range(cfg.n_layers):
        kp = np.zeros((pool_blocks, kvh, bs, hd), np.float16)
        vp = np.zeros((pool_blocks, kvh, bs, hd), np.float16)
        for b in range(len(cached)):
            for t in range(cached[b]):
                kp[tables[b, t // bs], :, t % bs] = ks[l][b][t]
                vp[tables[b, t // bs], :, t % bs] = vs[l][b][t]
        native.state.write(native.state_offsets[2 * l], kp)
        native.state.write(native.state_offsets[2 * l + 1], vp)


def test_batched_loop_equals_sequential_loops_and_the_oracle(oracle):
    cfg = DecoderConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ffn=1024, vocab=1024)
    B, N, max_ctx, bs = 3, 6, 64, cfg.block_size
    rng = np.random.default_rng(11)
    cached = np.array([0, 14, 37], np.int32)        # 14 -> crosses a page boundary during the loop
    first = rng.integers(0, cfg.vocab, B).astype(np.int32)
    max_blocks = max_ctx // bs
    tables = rng.permutation(B * max_blocks).astype(np.int32).reshape(B, max_blocks)
    specs = decoder_weights(cfg, 1)
    weights = make_decoder_weights(oracle, specs, seed=3)
    kvh, hd = cfg.n_kv_heads, cfg.head_dim
    ks = [[rng.standard_normal((cached[b], kvh, hd)).astype(np.float16) for b in range(B)] for _ in range(cfg.n_layers)]
    vs = [[rng.standard_normal((cached[b], kvh, hd)).astype(np.float16) for b in range(B)] for _ in range(cfg.n_layers)]

    # ---- the batch
    native = Native.load(weights)
    loop = DecodeLoop(native, cfg, B, max_ctx, tables)
    fill_pools(native, cfg, tables, ks, vs, cached)
    loop.begin(first, cached)
    batched_tokens, batched_logits = [], []
    for _ in range(N):
        loop.step()
        batched_tokens.append(loop.tokens())
        batched_logits.append(loop.logits())
    assert loop.steps == N and np.array_equal(loop.pos, cached + N)
    loop.free()
    native.close()
    batched_tokens = np.stack(batched_tokens)       # [N, B]

    # ---- one loop per sequence over its own part of the same pool layout
    for b in range(B):
        native = Native.load(weights)
        loop = DecodeLoop(native, cfg, 1, max_ctx, tables[b:b + 1])
        fill_pools(native, cfg, tables[b:b + 1], [[k[b]] for k in ks], [[v[b]] for v in vs], cached[b:b + 1])
        loop.begin(first[b:b + 1], cached[b:b + 1])
        for s in range(N):
            loop.step()
            assert loop.tokens()[0] == batched_tokens[s, b], (b, s)
            np.testing.assert_allclose(loop.logits()[0], batched_logits[s][b], rtol=0, atol=2e-3)
        loop.free()
        native.close()

    # ---- the oracle, one sequence at a time, fed the GPU's tokens
    worst, envelope = 0.0, 0.0
    for b in range(B):
        kb = [np.concatenate([ks[l][b], np.zeros((N, kvh, hd), np.float16)]) for l in range(cfg.n_layers)]
        vb = [np.concatenate([vs[l][b], np.zeros((N, kvh, hd), np.float16)]) for l in range(cfg.n_layers)]
        tok = first[b]
        for s in range(N):
            p = cached[b] + s
            view_k = [[kb[l][:p + 1]] for l in range(cfg.n_layers)]     # views: the oracle fills the new token's slot in place
            view_v = [[vb[l][:p + 1]] for l in range(cfg.n_layers)]
            want = oracle_decoder_step(oracle, cfg, specs, weights, np.array([tok], np.int32), np.array([p], np.int32), view_k, view_v)
            if s == 0:
                import copy
                noisy = oracle_decoder_step(NoisyOracle(oracle, 1e-6, b), cfg, specs, weights, np.array([tok], np.int32), np.array([p], np.int32),
                                            copy.deepcopy(view_k), copy.deepcopy(view_v))
                envelope = max(envelope, float(np.abs(noisy - want).max()))
            got = batched_logits[s][b]
            worst = max(worst, float(np.abs(got - want[0]).max()))
            top2 = np.sort(want[0])[-2:]
            if top2[1] - top2[0] > 0.1:
                assert int(want[0].argmax()) == batched_tokens[s, b], (b, s)
            tok = batched_tokens[s, b]
    print("decode loop: worst logits error against the oracle over %d steps %.3e (one-step noise envelope of the oracle %.3e)" % (N, worst, envelope))
    assert worst <= max(5e-2, 4 * envelope), (worst, envelope)
