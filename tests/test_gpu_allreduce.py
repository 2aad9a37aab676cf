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
