"""Small helpers shared by the GPU parity tests."""
import numpy as np

from tensorlisp_b200 import graph as G
from tensorlisp_b200.native import Native, NativeProgram


def close(got, want, tol):
    """The reference's own comparison (crates/tensorlisp/tests/native.rs:49-57):
    max|got-want| <= tol * max|want| + 1e-6."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if got.size == want.size:  # reads drop leading dimensions of extent 1
        got = got.reshape(want.shape)
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


class NoisyOracle:
    """The oracle with its mul_mat outputs perturbed: measures how far the reference's own arithmetic moves under a
    perturbation of the size a kernel makes. `eps` relative to each element (summation order: 1e-6), or, with
    `of_max`, relative to max|y| of the product (the folded-scale prompt kernel: its two f16 roundings per product
    leave an error of about 7e-5 of max|y| standard deviation, 3e-4 at most)."""

    def __init__(self, oracle, eps, seed, of_max=False):
        self.o, self.eps, self.r, self.of_max = oracle, eps, np.random.default_rng(seed), of_max

    def __getattr__(self, name):
        return getattr(self.o, name)

    def mul_mat(self, *a, **k):
        y = self.o.mul_mat(*a, **k)
        if self.of_max:
            return (y + self.eps * np.abs(y).max() * self.r.standard_normal(y.shape)).astype(np.float32)
        return (y * (1 + self.eps * self.r.standard_normal(y.shape))).astype(np.float32)


# ------------------------------------------------------------------ oracle-side decoder step
def make_decoder_weights(oracle, specs, seed=0):
    """N(0, 0.02) f32 matrices quantized with the oracle (bit-exact with the reference), norm weights N(1, 0.1)."""
    rng = np.random.default_rng(seed)
    out = []
    for s in specs:
        if len(s.ne) == 1:
            out.append((1 + 0.1 * rng.standard_normal(s.ne[0])).astype(np.float32))
        else:
            w = (rng.standard_normal((s.ne[1], s.ne[0])) * 0.02).astype(np.float32)
            out.append(oracle.quantize(s.ty, w))
    return out


def oracle_decoder_step(oracle, cfg, specs, weights, ids, pos, ks, vs):
    """The decode step of tensorlisp_b200.programs.decoder_step restated with oracle calls only.
    ks[l][s], vs[l][s]: f16 [ctx_s, kv_heads, hd] INCLUDING the new token's slot (filled here).
    Returns logits f32 [batch, vocab]."""
    W = {s.name: (s, w) for s, w in zip(specs, weights)}
    B = len(ids)
    hd, heads, kvh = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads

    def lin(name, x):
        s, w = W[name]
        return oracle.mul_mat(s.ty, w, s.ne[0], x)

    s, w = W["token_embd"]
    x = oracle.get_rows(s.ty, w, cfg.d_model, ids)
    for l in range(cfg.n_layers):
        p = "blk.%d." % l
        h = oracle.rms_norm(x, cfg.eps, W[p + "attn_norm"][1])
        q, k, v = lin(p + "wq", h), lin(p + "wk", h), lin(p + "wv", h)
        q = oracle.rope(q.reshape(B, heads, hd), pos, hd, 2, cfg.rope_theta)
        k = oracle.rope(k.reshape(B, kvh, hd), pos, hd, 2, cfg.rope_theta)
        for b in range(B):
            ks[l][b][pos[b]] = k[b].astype(np.float16)
            vs[l][b][pos[b]] = v[b].reshape(kvh, hd).astype(np.float16)
        a16, _ = oracle.attention_decode(q.astype(np.float16), ks[l], vs[l], kvh, 1.0 / np.sqrt(hd))
        o = lin(p + "wo", a16.astype(np.float32).reshape(B, heads * hd))
        x = x + o
        h = oracle.rms_norm(x, cfg.eps, W[p + "ffn_norm"][1])
        m = oracle.silu_mul(lin(p + "ffn_gate", h), lin(p + "ffn_up", h))
        x = x + lin(p + "ffn_down", m)
    x = oracle.rms_norm(x, cfg.eps, W["output_norm"][1])
    return lin("output", x)


# ------------------------------------------------------------------ oracle-side prompt pass
def causal_attention(q, k16, v16, n_seqs, n_tokens, heads, kvh, hd):
    """q f32 [T, heads, hd], k16 / v16 f16 [T, kvh, hd] -> f32 [T, heads*hd], prompts independent."""
    out = np.zeros((n_seqs * n_tokens, heads, hd), np.float32)
    grp = heads // kvh
    mask = np.triu(np.full((n_tokens, n_tokens), -np.inf, np.float32), 1)
    for s in range(n_seqs):
        r = slice(s * n_tokens, (s + 1) * n_tokens)
        for h in range(heads):
            kk = k16[r, h // grp].astype(np.float32)
            vv = v16[r, h // grp].astype(np.float32)
            sc = q[r, h] @ kk.T / np.float32(np.sqrt(hd)) + mask
            p = np.exp(sc - sc.max(axis=1, keepdims=True))
            out[r, h] = (p / p.sum(axis=1, keepdims=True)) @ vv
    return out.reshape(n_seqs * n_tokens, heads * hd)


def oracle_prefill(oracle, cfg, specs, weights, ids, pos, n_seqs, n_tokens):
    W = {s.name: (s, w) for s, w in zip(specs, weights)}
    T = len(ids)
    hd, heads, kvh = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads

    def lin(name, x):
        s, w = W[name]
        return oracle.mul_mat(s.ty, w, s.ne[0], np.ascontiguousarray(x, np.float32))

    s, w = W["token_embd"]
    x = oracle.get_rows(s.ty, w, cfg.d_model, ids)
    for l in range(cfg.n_layers):
        p = "blk.%d." % l
        h = oracle.rms_norm(x, cfg.eps, W[p + "attn_norm"][1])
        q, k, v = lin(p + "wq", h), lin(p + "wk", h), lin(p + "wv", h)
        q = oracle.rope(q.reshape(T, heads, hd), pos, hd, 2, cfg.rope_theta)
        k = oracle.rope(k.reshape(T, kvh, hd), pos, hd, 2, cfg.rope_theta)
        a = causal_attention(q, k.astype(np.float16), v.reshape(T, kvh, hd).astype(np.float16), n_seqs, n_tokens, heads, kvh, hd)
        x = x + lin(p + "wo", a)
        h = oracle.rms_norm(x, cfg.eps, W[p + "ffn_norm"][1])
        x = x + lin(p + "ffn_down", oracle.silu_mul(lin(p + "ffn_gate", h), lin(p + "ffn_up", h)))
    last = np.arange(n_seqs) * n_tokens + n_tokens - 1
    x = oracle.rms_norm(np.ascontiguousarray(x[last]), cfg.eps, W["output_norm"][1])
    return lin("output", x)


def varied_rows(seed: int, n: int = 1024) -> np.ndarray:
    """Rows of very different character for the row quantizers: normal at scales from 1e-6 to 1e4, uniform, heavy-tailed,
    sparse, one-sided, constant, alternating signs, a ramp, blocks of zeros inside noise, values at f16's limits."""
    r = np.random.default_rng(seed)
    rows = []
    for scale in (1e-6, 1e-3, 0.02, 1.0, 37.0, 1e4):
        rows.append(r.standard_normal(n) * scale)
    rows.append(r.uniform(-1, 1, n))
    rows.append(r.standard_cauchy(n).clip(-1e4, 1e4))
    rows.append(r.standard_normal(n) * (r.random(n) < 0.05))
    rows.append(np.abs(r.standard_normal(n)))
    rows.append(-np.abs(r.standard_normal(n)) - 3.0)
    rows.append(np.full(n, -0.75))
    rows.append(np.where(np.arange(n) % 2 == 0, 1.0, -1.0) * r.random(n))
    rows.append(np.linspace(-5, 5, n))
    z = r.standard_normal(n)
    z[64:128] = 0.0
    z[256:512] = 0.0
    rows.append(z)
    rows.append(r.choice([65504.0, -65504.0, 6e-8, -6e-8, 1.0], n))
    rows.append(r.standard_normal(n) * np.exp(r.uniform(-8, 8, n)))
    rows.append(np.round(r.standard_normal(n) * 3))         # many exact ties
    return np.asarray(rows, np.float32)


def write_safetensors(path, tensors) -> None:
    """A .safetensors file from {name: array}; bf16 tensors are given as ("BF16", uint16 array)."""
    import json
    import struct
    names = {np.dtype(np.float64): "F64", np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.int64): "I64",
             np.dtype(np.int32): "I32", np.dtype(np.int16): "I16", np.dtype(np.int8): "I8", np.dtype(np.uint8): "U8", np.dtype(np.bool_): "BOOL"}
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        if isinstance(a, tuple):
            st, a = a
        else:
            st = names[a.dtype]
        b = np.ascontiguousarray(a).tobytes()
        header[name] = {"dtype": st, "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))
