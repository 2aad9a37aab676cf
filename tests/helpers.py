"""Small helpers shared by the GPU parity tests."""
import numpy as np

from tensorlisp_b200 import graph as G
from tensorlisp_b200.native import Native, NativeProgram


def close(got, want, tol):
    """The reference's own comparison (crates/tensorlisp/tests/native.rs:49-57):
    max|got-want| <= tol * max|want| + 1e-6."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    err = np.abs(got - want).max() if got.size else 0.0
    bound = tol * (np.abs(want).max() if want.size else 0.0) + 1e-6
    assert err <= bound, "max error %.3e exceeds %.3e" % (err, bound)
    return err


class Model:
    """Weights + states + one compiled program, the way Model::load / run_entry drive the native
    executor (crates/tensorlisp/src/model.rs:454-518, 1041-1093)."""

    def __init__(self, graph: G.Graph, weights=(), state_bytes=(), outputs=None):
        self.native = Native.load([np.ascontiguousarray(w) for w in weights])
        self.native.alloc_states(list(state_bytes))
        self.graph = graph
        self.program = NativeProgram.compile(self.native, graph, outputs)

    def run(self, *inputs, state=None):
        for i, x in enumerate(inputs):
            self.program.set_input(i, x)
        self.program.run(state)
        return [a for _, a in self.program.outputs()]

    def close(self):
        self.program.free()
        self.native.close()
