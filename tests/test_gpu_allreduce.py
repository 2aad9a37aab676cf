"""The peer-memory all-reduce of the tensor-parallel path, checked on ONE GPU: the ranks are emulated
inside one cooperative launch (ranks that wait on one another may not be separate launches on one
device), each with its own exchange buffer. Every rank must end with the sum taken in rank order,
bit for bit the same on all ranks, over several calls in a row (slots alternate by parity, sequence
numbers only grow)."""
import ctypes as C

import numpy as np
import pytest

from tensorlisp_b200._lib import check, lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("n", [4, 4000, 32 * 4096, 262144])
def test_one_shot_allreduce_emulated(native, ranks, n):
    calls = 5
    rng = np.random.default_rng(ranks * 1000 + n)
    x = rng.standard_normal((ranks, n)).astype(np.float32)
    out = np.zeros_like(x)
    check(lib().tlb_comm_p2p_selftest(native.dev, ranks, n, calls, 0, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)))
    scaled = (x * np.float32(calls)).astype(np.float32)     # the last call's inputs
    want = scaled[0].copy()
    for r in range(1, ranks):
        want = (want + scaled[r]).astype(np.float32)        # rank order, f32
    for r in range(ranks):
        assert np.array_equal(out[r], want), r


@pytest.mark.parametrize("ranks,splits", [(2, 4), (8, 3), (4, 7)])
def test_exchange_behind_a_k_split(native, ranks, splits):
    """Every rank's input is the sum of `splits` partial results (the row-parallel mul_mat's K split),
    added in split order by the same kernel before the exchange."""
    n, calls = 32 * 4096, 3
    rng = np.random.default_rng(ranks * 10 + splits)
    x = rng.standard_normal((ranks, splits, n)).astype(np.float32)
    out = np.zeros((ranks, n), np.float32)
    check(lib().tlb_comm_p2p_selftest(native.dev, ranks, n, calls, splits, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)))
    scaled = (x * np.float32(calls)).astype(np.float32)
    per_rank = scaled[:, 0].copy()
    for s in range(1, splits):
        per_rank = (per_rank + scaled[:, s]).astype(np.float32)
    want = per_rank[0].copy()
    for r in range(1, ranks):
        want = (want + per_rank[r]).astype(np.float32)
    for r in range(ranks):
        assert np.array_equal(out[r], want), r


@pytest.mark.parametrize("flagged", ["0", "1"])
@pytest.mark.parametrize("ranks,splits", [(2, 1), (4, 4), (3, 2)])
def test_exchange_fused_with_add_norm_quant(native, oracle, ranks, splits, flagged, monkeypatch):
    """Both protocols of the fused exchange (TLB_XR_FLAGGED: every value in one 8-byte word with the call's sequence
    number, or plain values behind a system fence and one flag per rank and row). The exchange behind a row-parallel projection fused with the residual add, the RMS norm and the Q8_K
    quantizer of the next mul_mat (emulated ranks, one cooperative launch): the new residual stream is the
    exact f32 sum in split, then rank, order on every rank; the Q8_K block is the oracle's quantization of
    the oracle's norm of that stream (codes may differ by one where the sum of squares was added up in
    another order)."""
    monkeypatch.setenv("TLB_XR_FLAGGED", flagged)
    rows, K, calls, eps = 32, 4096, 3, 1e-5
    rng = np.random.default_rng(ranks * 7 + splits)
    x = (rng.standard_normal((ranks, splits, rows, K)) * 0.5).astype(np.float32)
    resid = rng.standard_normal((rows, K)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    al = lambda v: (v + 255) // 256 * 256
    d_off = al(rows * K)
    bsum_off = d_off + al(rows * (K // 256) * 4)
    act_bytes = bsum_off + al(rows * (K // 16) * 2)
    out_sum = np.zeros((ranks, rows, K), np.float32)
    out_q = np.zeros((ranks, act_bytes), np.uint8)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    check(lib().tlb_comm_p2p_selftest_rows(native.dev, ranks, rows, K, splits, calls, p(x), p(resid), p(w), eps, p(out_sum), p(out_q), act_bytes))
    scaled = (x * np.float32(calls)).astype(np.float32)
    per_rank = scaled[:, 0].copy()
    for s in range(1, splits):
        per_rank = (per_rank + scaled[:, s]).astype(np.float32)
    total = per_rank[0].copy()
    for r in range(1, ranks):
        total = (total + per_rank[r]).astype(np.float32)
    want_sum = (resid + total).astype(np.float32)
    want_q = oracle.quantize_q8_K(oracle.rms_norm(want_sum, eps, w)).reshape(rows, K // 256, 292)   # f32 d, 256 codes, 16 sums
    want_d = want_q[:, :, :4].copy().view(np.float32).reshape(rows, K // 256)
    want_codes = want_q[:, :, 4:260].copy().view(np.int8).reshape(rows, K)
    for r in range(ranks):
        assert np.array_equal(out_sum[r], want_sum), r
        codes = out_q[r, :rows * K].view(np.int8).reshape(rows, K)
        d = out_q[r, d_off:d_off + rows * (K // 256) * 4].view(np.float32).reshape(rows, K // 256)
        bs = out_q[r, bsum_off:bsum_off + rows * (K // 16) * 2].view(np.int16).reshape(rows, K // 16)
        assert np.allclose(d, want_d, rtol=2e-6, atol=0)
        diff = np.abs(codes.astype(np.int32) - want_codes.astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
        assert np.array_equal(bs, codes.reshape(rows, K // 16, 16).astype(np.int32).sum(axis=2).astype(np.int16))
        assert np.array_equal(out_q[r], out_q[0])    # every rank holds the same bytes


@pytest.mark.parametrize("ranks,absent", [(2, 1), (4, 0), (8, 5)])
def test_a_rank_that_never_arrives_ends_the_wait(native, ranks, absent):
    """One emulated rank never pushes. The waits of the others are bounded: after `spin_limit` probes they
    give up, the launch ends (nothing is left waiting on the device), the call reports Execution with the
    "gave up waiting" message that tlb_program_run gives for a real missing rank, and the device is usable
    afterwards (a complete exchange right behind it succeeds)."""
    import time
    from tensorlisp_b200._lib import TLB_EXECUTION
    n = 32 * 4096
    x = np.ones((ranks, n), np.float32)
    out = np.zeros_like(x)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    t0 = time.time()
    st = lib().tlb_comm_p2p_selftest_absent(native.dev, ranks, n, absent, 2000, p(x), p(out))
    assert st == TLB_EXECUTION, st
    assert b"gave up waiting" in lib().tlb_last_error()
    assert time.time() - t0 < 5.0
    check(lib().tlb_comm_p2p_selftest(native.dev, ranks, n, 2, 0, p(x), p(out)))
    assert np.array_equal(out, np.full_like(out, 2.0 * ranks))


@pytest.mark.parametrize("flagged", ["0", "1"])
def test_a_rank_that_never_arrives_ends_the_fused_exchange(native, flagged, monkeypatch):
    from tensorlisp_b200._lib import TLB_EXECUTION
    monkeypatch.setenv("TLB_XR_FLAGGED", flagged)
    ranks, rows, K, eps = 4, 32, 4096, 1e-5
    x = np.ones((ranks, 1, rows, K), np.float32)
    resid = np.ones((rows, K), np.float32)
    w = np.ones(K, np.float32)
    al = lambda v: (v + 255) // 256 * 256
    act_bytes = al(rows * K) + al(rows * (K // 256) * 4) + al(rows * (K // 16) * 2)
    out_sum = np.zeros((ranks, rows, K), np.float32)
    out_q = np.zeros((ranks, act_bytes), np.uint8)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    st = lib().tlb_comm_p2p_selftest_rows_absent(native.dev, ranks, rows, K, 2, 2000, p(x), p(resid), p(w), eps, p(out_sum), p(out_q), act_bytes)
    assert st == TLB_EXECUTION, st
    assert b"gave up waiting" in lib().tlb_last_error()
    check(lib().tlb_comm_p2p_selftest_rows(native.dev, ranks, rows, K, 1, 1, p(x), p(resid), p(w), eps, p(out_sum), p(out_q), act_bytes))
    assert np.array_equal(out_sum, np.full_like(out_sum, 1.0 + ranks))
