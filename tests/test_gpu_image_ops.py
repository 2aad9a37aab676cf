"""IM2COL, UPSCALE, POOL_2D, CONV_2D_DW, PAD and PAD_REFLECT_1D through compiled programs against the reference's own ggml
CPU operators on the same inputs (the build of the reference's vendored ggml under oracle/_ref; the reference's executor
has these as one-thread-per-element kernels: crates/kernels/src/cuda/native/core.cu:240-261, 285-358, 405-427, 483-536).
Copies and maxima are compared for equality, interpolations and sums to 1e-5 of max|want|."""
import numpy as np
import pytest

from helpers import close
from tensorlisp_b200 import graph as G
from tensorlisp_b200.native import Native, NativeProgram
from test_graph_ir import build_both, image_ops_program

pytestmark = pytest.mark.gpu


def test_image_ops_match_ggml(ref):
    named = []

    def prog(b):
        named.extend(image_ops_program(b))

    g, rg, pairs = build_both(ref, prog)
    rng = np.random.default_rng(7)
    inputs = {}
    for a, b in pairs:
        T = g.tensors[a]
        if T.storage_kind == G.INPUT:
            dt = np.float16 if T.ty == G.F16 else np.float32
            data = rng.standard_normal(T.ne[::-1]).astype(dt)
            inputs[T.storage_index] = data
            rg.write(b, data)
    outs = [pair for _, pair in named]
    for a, _ in outs:
        g.output(a)
    rg.compute([b for _, b in outs])
    n = Native.load([])
    n.alloc_states([])
    prog_gpu = NativeProgram.compile(n, g, [(name, a) for name, (a, _) in named])
    for i, data in inputs.items():
        prog_gpu.set_input(i, data)
    prog_gpu.run()
    got = dict(prog_gpu.outputs())
    for name, (a, b) in named:
        T = g.tensors[a]
        want = rg.read(b, np.float16 if T.ty == G.F16 else np.float32).astype(np.float32)
        have = np.asarray(got[name], np.float32).reshape(want.shape)
        if name.startswith(("pad", "im2col", "pool max")) or name in ("upscale mode 0", "upscale x2"):
            assert np.array_equal(have, want), name
        else:
            err = close(have, want, 1e-5)
            print("%s: max error %.2e of max|want|" % (name, err / max(np.abs(want).max(), 1e-30)))
    prog_gpu.free()
    n.close()
    rg.close()


def test_unsupported_image_parameters_fail_by_name():
    from tensorlisp_b200._lib import TlbError
    g = G.Graph()
    x = g.input(G.F32, [8, 8, 2, 1], "img")
    node = g.pad_ext(x, 1, 1, 0, 0, 0, 0, 0, 0)
    g.tensors[node].op_params[8] = 1     # circular padding
    g.output(node)
    n = Native.load([])
    n.alloc_states([])
    with pytest.raises(TlbError) as e:
        NativeProgram.compile(n, g)
    assert "PAD" in str(e.value) and "circular" in str(e.value)
    n.close()
