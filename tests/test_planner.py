"""Invariants of the arena planner on random graphs, without a GPU (the planner alone through tlb_plan_only).
The reference checks the same on 200 random graphs (crates/kernels/src/plan.rs:191-315): tensors that are live at the
same time never share bytes, so a node never writes over a source it reads; a view keeps its root alive; kept tensors
stay valid to the end; scratch blocks share nothing with anything live while they live; inputs, weights and states
resolve to their own buffers."""
import ctypes as C

import numpy as np

from tensorlisp_b200 import _lib
from tensorlisp_b200 import graph as G

ARENA, IO, STATE, WEIGHTS = 3, 2, 1, 0


def random_graph(rng):
    g = G.Graph()
    shapes = [[int(rng.integers(1, 9)) * 32, int(rng.integers(1, 5))] for _ in range(3)]
    pool = {i: [] for i in range(len(shapes))}          # tensors by shape
    for i, ne in enumerate(shapes):
        pool[i].append(g.input(G.F32, ne, "in%d" % i))
        if rng.random() < 0.5:
            pool[i].append(g.weight(G.F32, ne, "w%d" % i))
        if rng.random() < 0.3:
            pool[i].append(g.state(G.F32, ne, "s%d" % i))
    n_nodes = int(rng.integers(4, 40))
    for _ in range(n_nodes):
        i = int(rng.integers(0, len(shapes)))
        a = int(rng.choice(pool[i]))
        kind = rng.random()
        if kind < 0.45:
            b = int(rng.choice(pool[i]))
            t = g.add(a, b) if rng.random() < 0.5 else g.mul(a, b)
        elif kind < 0.65:
            t = g.scale(a, 2.0)
        elif kind < 0.8:
            # a view op: aliases its source (and, for views of views, the root)
            t = g.reshape(a, [shapes[i][0] // 2, shapes[i][1] * 2])
            t = g.reshape(t, shapes[i])
        elif kind < 0.9:
            t = g.cont(g.transpose(g.reshape(a, [shapes[i][0], shapes[i][1]])))
            t = g.reshape(t, shapes[i])
        else:
            t = g.sqr(a)
        pool[i].append(t)
    temps = [t for t in g.nodes if g.tensors[t].storage_kind == G.TEMP]
    for t in rng.choice(temps, size=min(len(temps), int(rng.integers(1, 4))), replace=False):
        g.output(int(t))
    return g


def plan(g, scratch):
    n, nn = len(g.tensors), len(g.nodes)
    cg, keep = g.to_c()
    wb = (C.c_uint32 * max(g.n_weights, 1))(*([0] * g.n_weights))
    wo = (C.c_uint64 * max(g.n_weights, 1))(*[4096 * i for i in range(g.n_weights)])
    so = (C.c_uint64 * max(g.n_states, 1))(*[8192 * i for i in range(g.n_states)])
    leaves = _lib.tlb_leaves(wb, wo, g.n_weights, so, g.n_states)
    sc = (C.c_uint64 * max(nn, 1))(*scratch)
    arena, io = C.c_uint64(), C.c_uint64()
    buf = (C.c_uint8 * max(n, 1))()
    off = (C.c_uint64 * max(n, 1))()
    soff = (C.c_int64 * max(nn, 1))()
    _lib.check(_lib.lib().tlb_plan_only(C.byref(cg), C.byref(leaves), sc, C.byref(arena), C.byref(io), buf, off, soff))
    del keep
    return arena.value, io.value, list(buf[:n]), list(off[:n]), list(soff[:nn])


def root_of(g, t):
    T = g.tensors[t]
    return T.view_src if T.view_src >= 0 else t


def test_random_graphs():
    rng = np.random.default_rng(20)
    checked_pairs = 0
    for it in range(200):
        g = random_graph(rng)
        nn = len(g.nodes)
        scratch = [int(rng.integers(1, 5000)) if rng.random() < 0.3 else 0 for _ in range(nn)]
        arena, io, buf, off, soff = plan(g, scratch)
        # liveness of every root, in node positions, the way a reader of the graph sees it
        first, last = {}, {}
        for pos, t in enumerate(g.nodes):
            for x in [t] + [s for s in g.tensors[t].src if s >= 0]:
                r = root_of(g, x)
                first.setdefault(r, pos)
                last[r] = pos
        for t in g.keep:
            last[root_of(g, t)] = nn
        blocks = []   # (first, last, offset, bytes, what)
        for r in first:
            R = g.tensors[r]
            if R.storage_kind == G.TEMP:
                assert buf[r] == ARENA and off[r] % 256 == 0
                assert off[r] + R.nbytes() <= arena
                blocks.append((first[r], last[r], off[r], R.nbytes(), "tensor %d" % r))
        for pos, want in enumerate(scratch):
            if want:
                assert soff[pos] >= 0 and soff[pos] % 256 == 0 and soff[pos] + want <= arena
                blocks.append((pos, min(pos + 2, nn - 1), soff[pos], want, "scratch of node %d" % pos))
            else:
                assert soff[pos] == -1
        for i in range(len(blocks)):
            for j in range(i + 1, len(blocks)):
                a, b = blocks[i], blocks[j]
                if a[0] <= b[1] and b[0] <= a[1]:      # live at the same time
                    checked_pairs += 1
                    assert a[2] + a[3] <= b[2] or b[2] + b[3] <= a[2], (it, a, b)
        # a node never writes over a source it reads (unless it IS a view of it)
        for t in g.nodes:
            T = g.tensors[t]
            if T.op in ("RESHAPE", "VIEW", "TRANSPOSE", "PERMUTE"):
                continue
            rt = root_of(g, t)
            for s in T.src:
                if s >= 0 and root_of(g, s) != rt and buf[rt] == ARENA and buf[root_of(g, s)] == ARENA:
                    rs = root_of(g, s)
                    assert off[rt] + g.tensors[rt].nbytes() <= off[rs] or off[rs] + g.tensors[rs].nbytes() <= off[rt]
        # views resolve to their root's place plus their offset; leaves to their own buffers
        ins = []
        for t, T in enumerate(g.tensors):
            r = root_of(g, t)
            assert buf[t] == buf[r] and off[t] == off[r] + (T.view_offs if T.view_src >= 0 else 0)
            if T.view_src < 0 and T.storage_kind == G.WEIGHT:
                assert buf[t] == WEIGHTS and off[t] == 4096 * T.storage_index
            if T.view_src < 0 and T.storage_kind == G.STATE:
                assert buf[t] == STATE and off[t] == 8192 * T.storage_index
            if T.view_src < 0 and T.storage_kind == G.INPUT:
                assert buf[t] == IO
                ins.append((off[t], T.nbytes()))
        ins.sort()
        for (o0, n0), (o1, _) in zip(ins, ins[1:]):
            assert o0 + n0 <= o1
        assert not ins or ins[-1][0] + ins[-1][1] <= io
    assert checked_pairs > 2000


def test_kept_tensor_is_not_reused():
    g = G.Graph()
    x = g.input(G.F32, [64, 4], "x")
    a = g.output(g.sqr(x))            # kept: must survive everything after it
    b = g.scale(x, 3.0)
    c = g.sqr(b)
    d = g.output(g.add(c, b))
    arena, io, buf, off, _ = plan(g, [0] * len(g.nodes))
    n = g.tensors[a].nbytes()
    for t in (b, c, d):
        assert off[a] + n <= off[t] or off[t] + g.tensors[t].nbytes() <= off[a]


def test_a_dead_tensor_is_reused():
    g = G.Graph()
    x = g.input(G.F32, [64, 4], "x")
    t = g.sqr(x)
    for _ in range(10):
        t = g.scale(t, 2.0)
    g.output(t)
    arena, *_ = plan(g, [0] * len(g.nodes))
    assert arena <= 3 * 1024       # a chain needs two live buffers at a time, not eleven
