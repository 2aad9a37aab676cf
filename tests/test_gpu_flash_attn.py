"""FLASH_ATTN_EXT (dense attention, reference lower.rs:575-657) against (a) the closed form
softmax(scale q k^T + slope mask) v in f64 on the same f16-rounded K/V, and (b) where the reference's
own ggml build travels with the repository, ggml's CPU flash_attn_ext with f32 K/V (the f32-accumulator
mode). Ragged query / key counts, GQA, a causal f16 mask with -inf, a per-head mask, soft cap, ALiBi."""
import numpy as np
import pytest

from helpers import Model, close
from tensorlisp_b200 import graph as G

pytestmark = pytest.mark.gpu
TOL = 1e-3


def closed_form(q, k, v, mask, scale, softcap=0.0, max_bias=0.0):
    """q [nb, nh, nq, d], k/v [nb, nhkv, nkv, d], mask [nb or 1, nh or 1, nq_pad, nkv] -> [nb, nq, nh, d]"""
    nb, nh, nq, d = q.shape
    nhkv = k.shape[1]
    out = np.zeros((nb, nq, nh, d))
    n2 = 1
    while n2 * 2 <= nh:
        n2 *= 2
    m0, m1 = 2.0 ** (-max_bias / n2), 2.0 ** (-(max_bias / 2) / n2)
    for b in range(nb):
        for h in range(nh):
            hk = h // (nh // nhkv)
            s = q[b, h].astype(np.float64) @ k[b, hk].astype(np.float64).T * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            if mask is not None:
                slope = 1.0 if max_bias <= 0 else (m0 ** (h + 1) if h < n2 else m1 ** (2 * (h - n2) + 1))
                s = s + slope * mask[b % mask.shape[0], h % mask.shape[1], :nq].astype(np.float64)
            s = s - s.max(axis=1, keepdims=True)
            p = np.exp(s)
            out[b, :, h] = (p / p.sum(axis=1, keepdims=True)) @ v[b, hk].astype(np.float64)
    return out.astype(np.float32)


def run_gpu(q, k, v, mask, scale, softcap, max_bias, kv_ty):
    nb, nh, nq, d = q.shape
    nhkv, nkv = k.shape[1], k.shape[2]
    g = G.Graph()
    tq = g.input(G.F32, [d, nq, nh, nb], "q")
    tk = g.input(kv_ty, [d, nkv, nhkv, nb], "k")
    tv = g.input(kv_ty, [d, nkv, nhkv, nb], "v")
    ins = [q, k, v]
    tm = None
    if mask is not None:
        tm = g.input(G.F16, [nkv, mask.shape[2], mask.shape[1], mask.shape[0]], "mask")
        ins.append(mask)
    y = g.output(g.flash_attn_ext(tq, tk, tv, tm, scale, max_bias, softcap, "attn"))
    m = Model(g)
    (got,) = m.run(*ins)
    m.close()
    return got.reshape(nb, nq, nh, d)


CASES = [
    # d, nq, nkv, nh, nhkv, nb, mask kind, softcap, max_bias, kv type
    (128, 70, 200, 8, 2, 2, "causal", 0.0, 0.0, G.F16),
    (128, 1, 333, 4, 4, 1, None, 0.0, 0.0, G.F16),
    (64, 130, 130, 4, 1, 1, "causal", 0.0, 0.0, G.F32),
    (128, 33, 96, 8, 8, 1, "per_head", 30.0, 0.0, G.F16),
    (64, 17, 64, 6, 2, 2, "causal", 0.0, 8.0, G.F16),
]


def make_case(case):
    d, nq, nkv, nh, nhkv, nb, mk, softcap, max_bias, kv_ty = case
    rng = np.random.default_rng(d + nq + nkv)
    q = rng.standard_normal((nb, nh, nq, d)).astype(np.float32)
    kdt = np.float16 if kv_ty == G.F16 else np.float32
    k = rng.standard_normal((nb, nhkv, nkv, d)).astype(kdt)
    v = rng.standard_normal((nb, nhkv, nkv, d)).astype(kdt)
    mask = None
    nq_pad = (nq + 31) // 32 * 32
    if mk == "causal":   # query i sees keys 0 .. nkv - nq + i
        mask = np.full((1, 1, nq_pad, nkv), -np.inf, np.float16)
        for i in range(nq):
            mask[0, 0, i, :nkv - nq + i + 1] = 0
    elif mk == "per_head":
        mask = (rng.standard_normal((nb, nh, nq_pad, nkv)) * 2).astype(np.float16)
        mask[:, :, :, ::7] = -np.inf
    return q, k, v, mask, 1.0 / np.sqrt(d), softcap, max_bias, kv_ty


@pytest.mark.parametrize("case", CASES, ids=[str(c[:6]) for c in CASES])
def test_flash_attn_closed_form(case):
    q, k, v, mask, scale, softcap, max_bias, kv_ty = make_case(case)
    got = run_gpu(q, k, v, mask, scale, softcap, max_bias, kv_ty)
    # the kernel rounds q to f16, as the CPU backend does with an f16 cache
    want = closed_form(q.astype(np.float16), k, v, mask, scale, softcap, max_bias)
    close(got, want, TOL)


def test_flash_attn_against_ggml(ref):
    """The reference's own ggml (f32 K/V so that it accumulates in f32; GGML_PREC_F32)."""
    from oracle.bindings import RefGraph, F32 as RF32, F16 as RF16
    case = CASES[0]
    q, k, v, mask, scale, softcap, max_bias, kv_ty = make_case(case)
    nb, nh, nq, d = q.shape
    nhkv, nkv = k.shape[1], k.shape[2]
    g = RefGraph(ref, 256 << 20, 8)
    tq = g.tensor(RF32, [d, nq, nh, nb], "q", q)
    tk = g.tensor(RF32, [d, nkv, nhkv, nb], "k", k.astype(np.float32))
    tv = g.tensor(RF32, [d, nkv, nhkv, nb], "v", v.astype(np.float32))
    tm = g.tensor(RF16, [nkv, mask.shape[2], 1, 1], "m", mask)
    o = g.op("flash_attn_ext", [tq, tk, tv, tm], ints=[10], floats=[scale, 0.0, 0.0])
    g.compute([o])
    want = g.read(o).reshape(nb, nq, nh, d)
    g.close()
    got = run_gpu(q, k, v, mask, scale, softcap, max_bias, kv_ty)
    close(got, want, TOL)


OTHER_SIZES = [
    # d, dv, nq, nkv, nh, nhkv, nb, kv type: the shapes of the reference's own tests (crates/tensorlisp/tests/native.rs:283-346:
    # head sizes 256, 72, 80, 96, 112; one query over a long cache, query counts around 16, key counts around the tiles)
    (256, 256, 1, 1000, 4, 1, 1, G.F16), (256, 256, 1, 100, 4, 1, 1, G.F16), (256, 256, 5, 60, 4, 1, 1, G.F16), (256, 256, 40, 70, 4, 1, 1, G.F32),
    (72, 72, 16, 1, 4, 2, 2, G.F16), (72, 72, 17, 17, 4, 2, 2, G.F32), (72, 72, 100, 300, 4, 2, 2, G.F16), (80, 80, 33, 129, 4, 2, 2, G.F16),
    (96, 96, 20, 5000, 4, 2, 2, G.F16), (112, 112, 50, 33, 4, 2, 2, G.F16),
    # values of another size than keys, the largest size, and a size that is no multiple of 8
    (192, 128, 7, 90, 4, 2, 1, G.F16), (512, 512, 3, 77, 2, 1, 1, G.F16), (100, 60, 9, 40, 2, 2, 1, G.F32),
]


@pytest.mark.parametrize("case", OTHER_SIZES, ids=[str(c[:7]) for c in OTHER_SIZES])
def test_other_head_sizes(case):
    """Head sizes other than 64 / 128 (one CTA per query, as in the reference). The padding mask has holes inside the valid
    range and hides the last quarter of the keys, as the reference's tests do; for one query over 256 keys or more the keys
    are split into stretches and merged."""
    d, dv, nq, nkv, nh, nhkv, nb, kv_ty = case
    rng = np.random.default_rng(d + nq + nkv)
    kdt = np.float16 if kv_ty == G.F16 else np.float32
    q = rng.standard_normal((nb, nh, nq, d)).astype(np.float32)
    k = rng.standard_normal((nb, nhkv, nkv, d)).astype(kdt)
    v = rng.standard_normal((nb, nhkv, nkv, dv)).astype(kdt)
    nq_pad = (nq + 31) // 32 * 32
    valid = np.zeros(nkv, bool)
    valid[[j for j in range(max(1, nkv * 3 // 4)) if j % 3 != 1 or nkv < 3]] = True
    mask = np.ascontiguousarray(np.broadcast_to(np.where(valid, np.float16(0), np.float16(-np.inf)), (1, 1, nq_pad, nkv)))
    scale = 1.0 / np.sqrt(d)
    g = G.Graph()
    tq = g.input(G.F32, [d, nq, nh, nb], "q")
    tk = g.input(kv_ty, [d, nkv, nhkv, nb], "k")
    tv = g.input(kv_ty, [dv, nkv, nhkv, nb], "v")
    tm = g.input(G.F16, [nkv, nq_pad, 1, 1], "mask")
    g.output(g.flash_attn_ext(tq, tk, tv, tm, scale, 0.0, 0.0, "attn"))
    m = Model(g)
    (got,) = m.run(q, k, v, mask)
    m.close()
    got = got.reshape(nb, nq, nh, dv)
    qq = (q.astype(np.float16) if kv_ty == G.F16 else q).astype(np.float64)     # an f16 cache rounds the query to f16
    want = np.zeros((nb, nq, nh, dv))
    for b in range(nb):
        for h in range(nh):
            hk = h // (nh // nhkv)
            sc = qq[b, h] @ k[b, hk].astype(np.float64).T * scale + mask[0, 0, :nq].astype(np.float64)
            pr = np.exp(sc - sc.max(axis=1, keepdims=True))
            want[b, :, h] = (pr / pr.sum(axis=1, keepdims=True)) @ v[b, hk].astype(np.float64)
    close(got, want.astype(np.float32), TOL)


@pytest.mark.parametrize("name,ty,d", [("q8_0", G.Q8_0, 128), ("q4_0", G.Q4_0, 64), ("q5_1", G.Q5_1, 96), ("q4_K", G.Q4_K, 256), ("q6_K", G.Q6_K, 256),
                                       ("bf16", G.BF16, 128)])
def test_quantized_and_bf16_keys_and_values(oracle, name, ty, d):
    """The reference's lowering takes keys and values of every type it can decode (crates/kernels/src/cuda/lower.rs:587-589):
    a cache held as bf16 or as quantized blocks is decoded element by element, the query stays f32. Closed form on the
    decoded values."""
    nq, nkv, nh, nhkv, nb = 5, 70, 4, 2, 1
    rng = np.random.default_rng(d + ty)
    q = rng.standard_normal((nb, nh, nq, d)).astype(np.float32)
    k = rng.standard_normal((nb * nhkv * nkv, d)).astype(np.float32)
    v = rng.standard_normal((nb * nhkv * nkv, d)).astype(np.float32)
    kq, vq = oracle.quantize(ty, k), oracle.quantize(ty, v)
    if ty == G.BF16:
        dec = lambda b: (b.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(-1, d)
    else:
        dec = lambda b: oracle.dequantize(ty, b, d).reshape(-1, d)
    kd, vd = dec(kq).reshape(nb, nhkv, nkv, d), dec(vq).reshape(nb, nhkv, nkv, d)
    scale = 1.0 / np.sqrt(d)
    g = G.Graph()
    tk = g.weight(ty, [d, nkv, nhkv, nb], "k")
    tv = g.weight(ty, [d, nkv, nhkv, nb], "v")
    tq = g.input(G.F32, [d, nq, nh, nb], "q")
    g.output(g.flash_attn_ext(tq, tk, tv, None, scale, 0.0, 0.0, "attn"))
    m = Model(g, [kq, vq])
    (got,) = m.run(q)
    m.close()
    want = closed_form(q, kd, vd, None, scale)
    close(got.reshape(nb, nq, nh, d), want, TOL)


def test_sinks_are_reported_by_name():
    from tensorlisp_b200._lib import TlbError
    g = G.Graph()
    tq = g.input(G.F32, [128, 4, 2, 1], "q")
    tk = g.input(G.F16, [128, 8, 2, 1], "k")
    tv = g.input(G.F16, [128, 8, 2, 1], "v")
    y = g.flash_attn_ext(tq, tk, tv, None, 0.1, name="attn")
    g.tensors[y].src[4] = g.input(G.F32, [2], "sinks")
    g.output(y)
    with pytest.raises(TlbError) as e:
        Model(g)
    assert "FLASH_ATTN_EXT" in str(e.value) and "not implemented" in str(e.value)


def test_causal_prompt_2048_tokens():
    """The prompt-pass shape: 2048 queries over 2048 keys, 32 heads over 8 KV heads of 128, causal f16 mask. The kernel
    skips key tiles that the mask hides completely (most of the upper triangle); the closed form is evaluated on a
    sample of query rows of every head, which covers first / last rows of tiles and the diagonal tiles."""
    d, n, nh, nhkv = 128, 2048, 32, 8
    rng = np.random.default_rng(2048)
    q = rng.standard_normal((1, nh, n, d)).astype(np.float32)
    k = rng.standard_normal((1, nhkv, n, d)).astype(np.float16)
    v = rng.standard_normal((1, nhkv, n, d)).astype(np.float16)
    mask = np.triu(np.full((n, n), -np.inf, np.float16), 1).reshape(1, 1, n, n)
    scale = 1.0 / np.sqrt(d)
    got = run_gpu(q, k, v, mask, scale, 0.0, 0.0, G.F16)[0]          # [nq, nh, d]
    rows = sorted(set([0, 1, 63, 64, 65, 127, 128, 1023, 1024, 2047] + [int(i) for i in rng.integers(0, n, 54)]))
    q16 = q.astype(np.float16).astype(np.float64)
    worst = 0.0
    for h in range(nh):
        kk, vv = k[0, h // (nh // nhkv)].astype(np.float64), v[0, h // (nh // nhkv)].astype(np.float64)
        for i in rows:
            s = q16[0, h, i] @ kk[:i + 1].T * scale
            p = np.exp(s - s.max())
            want = (p / p.sum()) @ vv[:i + 1]
            worst = max(worst, float(np.abs(got[i, h] - want).max() / max(np.abs(want).max(), 1e-6)))
    assert worst <= TOL, worst


@pytest.mark.parametrize("nq,nkv,nh,nhkv,nb", [(1, 4000, 8, 2, 2), (3, 1111, 4, 4, 1), (1, 300, 32, 8, 1)])
def test_few_queries_over_a_long_cache_split_the_keys(nq, nkv, nh, nhkv, nb):
    """A one-query FLASH_ATTN_EXT over a long dense cache cuts the keys into stretches, one CTA each, and merges them with a
    second launch (the reference's split-KV decode, crates/kernels/src/cuda/native/fa.cu:114-231, lower.rs:764-779). The mask
    hides a tail of the cache (what a decode step over a preallocated dense cache passes). Checked against the closed form
    and against the same node with the split turned off (TL_NATIVE_FA=plain)."""
    import os
    d = 128
    rng = np.random.default_rng(nq + nkv)
    q = rng.standard_normal((nb, nh, nq, d)).astype(np.float32)
    k = rng.standard_normal((nb, nhkv, nkv, d)).astype(np.float16)
    v = rng.standard_normal((nb, nhkv, nkv, d)).astype(np.float16)
    nq_pad = (nq + 31) // 32 * 32
    mask = np.zeros((1, 1, nq_pad, nkv), np.float16)
    mask[..., nkv - nkv // 5:] = -np.inf
    scale = 1.0 / np.sqrt(d)
    got = run_gpu(q, k, v, mask, scale, 0.0, 0.0, G.F16)
    os.environ["TL_NATIVE_FA"] = "plain"
    try:
        plain = run_gpu(q, k, v, mask, scale, 0.0, 0.0, G.F16)
    finally:
        del os.environ["TL_NATIVE_FA"]
    want = closed_form(q.astype(np.float16), k, v, mask, scale, 0.0, 0.0)
    close(got, want, TOL)
    close(got, plain, 5e-4)     # P is rounded to f16 against a different running maximum in the two schedules
