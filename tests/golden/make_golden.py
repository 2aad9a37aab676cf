"""Generates tests/golden/golden.npz from the reference's OWN ggml build (oracle/_ref, variant
`base` = the reference's flags), so the fixtures travel to machines without a reference checkout.

    python tests/golden/make_golden.py

Every array is produced by the reference code: ggml_quantize_chunk, the CPU backend's activation
quantizers, and graphs computed by ggml's CPU backend through the public C API. Inputs are seeded
numpy draws and are stored next to the outputs.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.bindings import F16, F32, I32, Q4_0, Q4_K, Q8_0, Ref  # noqa: E402


def hard_rows(rng, rows, n):
    """Rows that exercise the quantizers' edge cases: all-zero and constant blocks, one huge outlier,
    all-positive / all-negative blocks, exact ties, tiny magnitudes."""
    x = (rng.standard_normal((rows, n)) * 0.02).astype(np.float32)
    x[0, :64] = 0.0
    x[0, 64:96] = 0.125
    x[1, 5] = 37.5
    x[1, 300] = -1e-6
    x[2] = np.abs(x[2])
    x[3] = -np.abs(x[3])
    x[4, :32] = np.tile(np.array([1.0, -1.0], np.float32), 16)
    x[5] *= 1e-6
    x[6, ::2] = 0.5
    x[6, 1::2] = -0.5
    x[7] = np.round(x[7] * 1000) / 1000
    return x


def main():
    ref = Ref("base")
    rng = np.random.default_rng(20240607)
    out = {}

    # ---- weight quantizers
    xq = np.concatenate([(rng.standard_normal((8, 512)) * 0.02).astype(np.float32), hard_rows(rng, 8, 512)])
    out["quant_x"] = xq
    for ty, nm in ((Q8_0, "q8_0"), (Q4_0, "q4_0"), (Q4_K, "q4_K")):
        out["quant_" + nm] = ref.quantize(ty, xq)
        out["dequant_" + nm] = ref.dequantize(ty, out["quant_" + nm], 512)

    # ---- activation quantizers of the CPU mul_mat
    xa = np.concatenate([rng.standard_normal((4, 512)).astype(np.float32), hard_rows(rng, 8, 512)])
    out["act_x"] = xa
    out["act_q8_0"] = ref.act_q8_0(xa)
    out["act_q8_K"] = ref.act_q8_K(xa)

    # ---- mul_mat through the CPU backend
    W = (rng.standard_normal((24, 512)) * 0.02).astype(np.float32)
    X = rng.standard_normal((5, 512)).astype(np.float32)
    out["mm_w"], out["mm_x"] = W, X
    for ty, nm in ((Q8_0, "q8_0"), (Q4_0, "q4_0"), (Q4_K, "q4_K")):
        g = ref.graph(64 << 20, 2)
        w = g.tensor(ty, [512, 24], data=ref.quantize(ty, W))
        x = g.tensor(F32, [512, 5], data=X)
        y = g.op("mul_mat", [w, x])
        g.compute([y])
        out["mm_y_" + nm] = g.read(y).reshape(5, 24).copy()
        g.close()

    # ---- row ops
    g = ref.graph(64 << 20, 2)
    xr = rng.standard_normal((6, 384)).astype(np.float32) * 3
    wr = (1 + 0.1 * rng.standard_normal(384)).astype(np.float32)
    ur = rng.standard_normal((6, 384)).astype(np.float32)
    out["row_x"], out["row_w"], out["row_u"] = xr, wr, ur
    x = g.tensor(F32, [384, 6], data=xr)
    w = g.tensor(F32, [384], data=wr)
    u = g.tensor(F32, [384, 6], data=ur)
    n = g.op("rms_norm", [x], floats=[1e-5])
    nm = g.op("mul", [n, w])
    n_only = g.op("rms_norm", [x], floats=[1e-6])
    si = g.op("mul", [g.op("unary", [x], ints=[10]), u])
    sw = g.op("glu_split", [x, u], ints=[2])
    sm = g.op("soft_max_ext", [x, None], floats=[0.25, 0.0])
    am = g.op("argmax", [x])
    g.compute([nm, n_only, si, sw, sm, am])
    out["row_rms_mul"] = g.read(nm).reshape(6, 384).copy()
    out["row_rms"] = g.read(n_only).reshape(6, 384).copy()
    out["row_silu_mul"] = g.read(si).reshape(6, 384).copy()
    out["row_swiglu"] = g.read(sw).reshape(6, 384).copy()
    out["row_softmax"] = g.read(sm).reshape(6, 384).copy()
    out["row_argmax"] = g.read(am, np.int32).copy()
    g.close()

    # ---- argmax ties: the last index wins on the CPU
    g = ref.graph(16 << 20, 1)
    ties = np.zeros((3, 40), np.float32)
    ties[0, [3, 17, 29]] = 2.0
    ties[1, :] = -1.0
    ties[2, 39] = 5.0
    ties[2, 0] = 5.0
    out["ties_x"] = ties
    t = g.tensor(F32, [40, 3], data=ties)
    a = g.op("argmax", [t])
    g.compute([a])
    out["ties_argmax"] = g.read(a, np.int32).copy()
    g.close()

    # ---- rope (neox and normal), positions up to 8191, theta 500000
    g = ref.graph(64 << 20, 2)
    xr = rng.standard_normal((5, 3, 128)).astype(np.float32)  # [tokens, heads, hd]
    pos = np.array([0, 1, 777, 4095, 8191], np.int32)
    out["rope_x"], out["rope_pos"] = xr, pos
    x = g.tensor(F32, [128, 3, 5], data=xr)
    p = g.tensor(I32, [5], data=pos)
    for mode, nm in ((2, "neox"), (0, "normal")):
        r = g.op("rope_ext", [x, p, None], ints=[128, mode, 0], floats=[500000.0, 1.0, 0.0, 1.0, 32.0, 1.0])
        g.compute([r])
        out["rope_" + nm] = g.read(r).reshape(5, 3, 128).copy()
    r = g.op("rope_ext", [x, p, None], ints=[64, 2, 0], floats=[10000.0, 1.0, 0.0, 1.0, 32.0, 1.0])
    g.compute([r])
    out["rope_neox_partial"] = g.read(r).reshape(5, 3, 128).copy()
    g.close()

    # ---- embedding lookup from a Q8_0 table
    g = ref.graph(64 << 20, 2)
    tab = (rng.standard_normal((50, 256)) * 0.02).astype(np.float32)
    ids = np.array([0, 49, 7, 7, 23], np.int32)
    out["emb_table"], out["emb_ids"] = tab, ids
    t = g.tensor(Q8_0, [256, 50], data=ref.quantize(Q8_0, tab))
    i = g.tensor(I32, [5], data=ids)
    e = g.op("get_rows", [t, i])
    g.compute([e])
    out["emb_rows"] = g.read(e).reshape(5, 256).copy()
    g.close()

    # ---- decode attention: dense K/V (f16 values held in f32 tensors => f32 accumulator on the CPU),
    # one query per sequence, GQA 4:1. q is f16-rounded, as the paged node takes f16 queries.
    seqs, heads, kvh, hs = 3, 8, 2, 128
    ctxs = [5, 37, 130]
    scale = 1.0 / np.sqrt(hs)
    q = rng.standard_normal((seqs, heads, hs)).astype(np.float16)
    out["att_q"] = q
    out["att_ctx"] = np.array(ctxs, np.int32)
    att = np.zeros((seqs, heads, hs), np.float32)
    for s, ctx in enumerate(ctxs):
        k = rng.standard_normal((ctx, kvh, hs)).astype(np.float16)
        v = rng.standard_normal((ctx, kvh, hs)).astype(np.float16)
        out["att_k%d" % s], out["att_v%d" % s] = k, v
        g = ref.graph(64 << 20, 2)
        # ggml layouts: q [hs, 1, heads], k/v [hs, ctx, kvh]
        tq = g.tensor(F32, [hs, 1, heads], data=q[s].astype(np.float32).reshape(heads, 1, hs))
        tk = g.tensor(F32, [hs, ctx, kvh], data=np.ascontiguousarray(k.astype(np.float32).transpose(1, 0, 2)))
        tv = g.tensor(F32, [hs, ctx, kvh], data=np.ascontiguousarray(v.astype(np.float32).transpose(1, 0, 2)))
        o = g.op("flash_attn_ext", [tq, tk, tv, None], ints=[10], floats=[scale, 0.0, 0.0])  # GGML_PREC_F32
        g.compute([o])
        att[s] = g.read(o).reshape(1, heads, hs)[0]
        g.close()
    out["att_out"] = att

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays; ref flags:", ref.build_flags())


if __name__ == "__main__":
    main()
