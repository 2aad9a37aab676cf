"""Bounded waits and graph-replay keys of the executor.

Every wait inside a kernel of the library (mbarrier waits of the TMA / tcgen05 kernels, flag waits of the peer-memory
exchange) has a probe limit, after which the kernel sets the device error word and returns, and tlb_program_run reports
Execution instead of hanging. The tests make such waits run out with a small limit; nothing is left waiting on the GPU."""
import ctypes as C

import numpy as np
import pytest

from tensorlisp_b200 import graph as G
from tensorlisp_b200._lib import TLB_EXECUTION, check, lib
from tensorlisp_b200.native import Native, NativeProgram

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nap", [0, 64])
def test_an_mbarrier_wait_that_nothing_completes_gives_up(native, nap):
    us = C.c_double(0)
    st = lib().tlb_selftest_wait_runs_out(native.dev, 2000, nap, C.byref(us))
    assert st == TLB_EXECUTION, st
    assert b"gave up waiting" in lib().tlb_last_error()
    # 2000 probes take milliseconds at most; the kernels' own limit (2^22 probes) is about 2000 times that
    assert 0 < us.value < 1e6, us.value
    print("2000 probes, %d ns naps: %.1f us (%.3f us per probe; 2^22 probes = %.2f s)" % (nap, us.value, us.value / 2000, us.value / 2000 * 4194304 / 1e6))
    # the device is usable afterwards
    check(lib().tlb_device_sync(native.dev))


def _two_launch_program(native):
    g = G.Graph()
    x = g.input(G.F32, [64, 4], "x")
    y = g.output(g.scale(g.sqr(x), 2.0))
    return NativeProgram.compile(native, g), y


def test_a_changed_communicator_is_not_replayed_from_an_old_graph():
    """The launches of a captured CUDA graph have the communicator's state baked in, so the key a graph is replayed
    under includes the communicator generation: after init / destroy the next run captures anew."""
    native = Native.load([])
    prog, y = _two_launch_program(native)
    x = np.arange(256, dtype=np.float32).reshape(4, 64)
    prog.set_input(0, x)
    L = lib()
    gen0 = L.tlb_device_comm_generation(native.dev)
    prog.run()
    prog.run()
    assert L.tlb_program_graph_count(prog.h) == 1
    check(L.tlb_comm_init(native.dev, 1, 0, None))
    assert L.tlb_device_comm_generation(native.dev) == gen0 + 1
    prog.run()
    assert L.tlb_program_graph_count(prog.h) == 2
    check(L.tlb_comm_destroy(native.dev))
    assert L.tlb_device_comm_generation(native.dev) == gen0 + 2
    prog.run()
    assert L.tlb_program_graph_count(prog.h) == 3
    assert np.array_equal(prog.read(y).reshape(4, 64), 2 * x * x)
    prog.free()
    native.close()


def test_a_second_device_in_the_same_process_runs_the_large_shared_memory_kernels(oracle):
    """The opt-in to more than 48 KB of dynamic shared memory is made per device: a program on ordinal 1 must run the
    TMA-streamed GEMV and the tcgen05 mul_mat just like one on ordinal 0."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    from oracle.bindings import Q4_K
    rng = np.random.default_rng(5)
    K, M = 1024, 256
    w = oracle.quantize(Q4_K, (rng.standard_normal((M, K)) * 0.02).astype(np.float32))
    for ordinal in (0, 1):
        for N in (2, 32):
            x = rng.standard_normal((N, K)).astype(np.float32)
            g = G.Graph()
            tw = g.weight(G.Q4_K, [K, M], "W")
            tx = g.input(G.F32, [K, N], "x")
            y = g.output(g.mul_mat(tw, tx, "y"))
            native = Native.load([w], ordinal=ordinal)
            prog = NativeProgram.compile(native, g)
            prog.set_input(0, x)
            prog.run()
            got = prog.read(y)
            want = oracle.mul_mat(Q4_K, w, K, x)
            assert np.abs(got.reshape(want.shape) - want).max() <= 1e-3 * np.abs(want).max()
            prog.free()
            native.close()
