"""TEST INFRASTRUCTURE ONLY: ctypes bindings for the two checkers.

* ``Oracle``  -- oracle/liboracle.so, the plain-C restatement (oracle/oracle.c).
* ``Ref``     -- oracle/_ref/libtlref_<variant>.so, the reference's own vendored ggml CPU backend
                 behind oracle/ref_harness.cpp (built by oracle/build.py from a reference checkout).

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
import this module. Nothing in the product package does.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

F32, F16, Q4_0, Q8_0, Q4_K, I32, I64 = 0, 1, 2, 8, 12, 26, 27
Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, Q6_K, BF16 = 3, 6, 7, 10, 11, 13, 14, 30   # quantized and decoded; mul_mat through exact dequantization

_p = C.c_void_p
_i64 = C.c_int64


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_p)


class Oracle:
    def __init__(self) -> None:
        so = HERE / "liboracle.so"
        if not so.exists():
            import importlib.util
            spec = importlib.util.spec_from_file_location("_orc_build", HERE / "build.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        L = C.CDLL(str(so))
        self.L = L
        L.orc_row_size.restype = _i64
        L.orc_row_size.argtypes = [C.c_int, _i64]
        L.orc_quantize_rows.argtypes = [C.c_int, _p, _i64, _i64, _p]
        L.orc_dequantize_row.argtypes = [C.c_int, _p, _p, _i64]
        L.orc_quantize_row_q8_K.argtypes = [_p, _p, _i64]
        L.orc_mul_mat.argtypes = [C.c_int, _p, _i64, _i64, _p, _i64, _p]
        L.orc_mul_mat_dequant.argtypes = [C.c_int, _p, _i64, _i64, _p, _i64, _p]
        L.orc_rms_norm.argtypes = [_p, _i64, _i64, C.c_float, _p, _p]
        L.orc_silu_mul.argtypes = [_p, _p, _i64, _p]
        L.orc_rope.argtypes = [_p, _i64, _i64, _i64, _p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, _p]
        L.orc_soft_max.argtypes = [_p, _i64, _i64, C.c_float, _p]
        L.orc_get_rows.argtypes = [C.c_int, _p, _i64, _p, _i64, _p]
        L.orc_argmax.argtypes = [_p, _i64, _i64, _p]
        L.orc_attention_decode.argtypes = [_p, _p, _p, _p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _p, _p]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]

    def row_size(self, ty: int, ne0: int) -> int:
        return int(self.L.orc_row_size(ty, ne0))

    def quantize(self, ty: int, x: np.ndarray) -> np.ndarray:
        """x: f32 [rows, n] -> uint8 [rows, row_size]."""
        x = np.ascontiguousarray(x, np.float32)
        rows, n = x.shape
        out = np.zeros((rows, self.row_size(ty, n)), np.uint8)
        assert self.L.orc_quantize_rows(ty, _ptr(x), rows, n, _ptr(out)) == 0
        return out

    def quantize_q8_K(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        rows, n = x.shape
        out = np.zeros((rows, n // 256 * 292), np.uint8)
        for r in range(rows):
            self.L.orc_quantize_row_q8_K(_ptr(x[r]), _ptr(out[r]), n)
        return out

    def dequantize(self, ty: int, q: np.ndarray, n: int) -> np.ndarray:
        q = np.ascontiguousarray(q)
        rows = q.shape[0]
        out = np.zeros((rows, n), np.float32)
        for r in range(rows):
            assert self.L.orc_dequantize_row(ty, _ptr(q[r]), _ptr(out[r]), n) == 0
        return out

    def mul_mat(self, ty: int, W: np.ndarray, K: int, x: np.ndarray, dequant: bool = False) -> np.ndarray:
        """W: [M, row bytes] (or f32/f16 [M, K]); x: f32 [N, K] -> f32 [N, M]."""
        W = np.ascontiguousarray(W)
        x = np.ascontiguousarray(x, np.float32)
        M, N = W.shape[0], x.shape[0]
        y = np.zeros((N, M), np.float32)
        f = self.L.orc_mul_mat_dequant if dequant else self.L.orc_mul_mat
        assert f(ty, _ptr(W), K, M, _ptr(x), N, _ptr(y)) == 0
        return y

    def rms_norm(self, x: np.ndarray, eps: float, w: np.ndarray | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        n = x.shape[-1]
        if w is not None:
            w = np.ascontiguousarray(w, np.float32)
        self.L.orc_rms_norm(_ptr(x), n, x.size // n, eps, _ptr(w) if w is not None else None, _ptr(y))
        return y

    def silu_mul(self, g: np.ndarray, u: np.ndarray) -> np.ndarray:
        g = np.ascontiguousarray(g, np.float32)
        u = np.ascontiguousarray(u, np.float32)
        y = np.empty_like(g)
        self.L.orc_silu_mul(_ptr(g), _ptr(u), g.size, _ptr(y))
        return y

    def rope(self, x: np.ndarray, pos: np.ndarray, n_dims: int, mode: int, freq_base: float,
             freq_scale: float = 1.0, attn_factor: float = 1.0) -> np.ndarray:
        """x: f32 [tokens, heads, ne0]."""
        x = np.ascontiguousarray(x, np.float32)
        pos = np.ascontiguousarray(pos, np.int32)
        tokens, heads, ne0 = x.shape
        y = np.empty_like(x)
        self.L.orc_rope(_ptr(x), ne0, heads, tokens, _ptr(pos), n_dims, mode, freq_base, freq_scale,
                        attn_factor, _ptr(y))
        return y

    def soft_max(self, x: np.ndarray, scale: float = 1.0) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        n = x.shape[-1]
        self.L.orc_soft_max(_ptr(x), n, x.size // n, scale, _ptr(y))
        return y

    def get_rows(self, ty: int, table: np.ndarray, ne0: int, ids: np.ndarray) -> np.ndarray:
        table = np.ascontiguousarray(table)
        ids = np.ascontiguousarray(ids, np.int32)
        y = np.zeros((ids.size, ne0), np.float32)
        assert self.L.orc_get_rows(ty, _ptr(table), ne0, _ptr(ids), ids.size, _ptr(y)) == 0
        return y

    def argmax(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        n = x.shape[-1]
        out = np.zeros(x.size // n, np.int32)
        self.L.orc_argmax(_ptr(x), n, x.size // n, _ptr(out))
        return out

    def attention_decode(self, q: np.ndarray, ks: list[np.ndarray], vs: list[np.ndarray], kv_heads: int,
                         scale: float) -> tuple[np.ndarray, np.ndarray]:
        """q: f16 [seqs, heads, hs]; ks[s], vs[s]: f16 [ctx_s, kv_heads, hs] -> (f16, f32) [seqs, heads, hs]."""
        q = np.ascontiguousarray(q, np.float16)
        seqs, heads, hs = q.shape
        ks = [np.ascontiguousarray(k, np.float16) for k in ks]
        vs = [np.ascontiguousarray(v, np.float16) for v in vs]
        kp = (C.c_void_p * seqs)(*[k.ctypes.data for k in ks])
        vp = (C.c_void_p * seqs)(*[v.ctypes.data for v in vs])
        ctx = np.array([k.shape[0] for k in ks], np.int32)
        out = np.zeros((seqs, heads, hs), np.float16)
        out32 = np.zeros((seqs, heads, hs), np.float32)
        self.L.orc_attention_decode(_ptr(q), kp, vp, _ptr(ctx), seqs, heads, kv_heads, hs, scale, _ptr(out),
                                    _ptr(out32))
        return out, out32


def _cpu_flags() -> set[str]:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def best_ref_variant() -> str | None:
    """The fastest reference build this host can execute (for the timed CPU baseline)."""
    flags = _cpu_flags()
    d = HERE / "_ref"
    if (d / "libtlref_v4.so").exists() and {"avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512_vnni"} <= flags:
        return "v4"
    if (d / "libtlref_v3.so").exists() and {"avx2", "fma", "f16c", "bmi2"} <= flags:
        return "v3"
    if (d / "libtlref_base.so").exists():
        return "base"
    return None


def ref_available(variant: str = "base") -> bool:
    return (HERE / "_ref" / ("libtlref_%s.so" % variant)).exists()


class Ref:
    """The reference's own ggml (variant 'base' = the canonical parity build)."""

    def __init__(self, variant: str = "base") -> None:
        so = HERE / "_ref" / ("libtlref_%s.so" % variant)
        if not so.exists():
            raise FileNotFoundError(str(so))
        L = C.CDLL(str(so))
        self.L = L
        self.variant = variant
        L.tlref_row_size.restype = _i64
        L.tlref_row_size.argtypes = [C.c_int, _i64]
        L.tlref_quantize.restype = _i64
        L.tlref_quantize.argtypes = [C.c_int, _p, _p, _i64, _i64]
        L.tlref_dequantize.argtypes = [C.c_int, _p, _p, _i64]
        L.tlref_act_q8_0.argtypes = [_p, _p, _i64]
        L.tlref_act_q8_K.argtypes = [_p, _p, _i64]
        L.tlref_new.restype = _p
        L.tlref_new.argtypes = [C.c_uint64, C.c_int]
        L.tlref_free.argtypes = [_p]
        L.tlref_error.restype = C.c_char_p
        L.tlref_error.argtypes = [_p]
        L.tlref_tensor.argtypes = [_p, C.c_int, _p, C.c_char_p]
        L.tlref_data.restype = _p
        L.tlref_data.argtypes = [_p, C.c_int]
        L.tlref_nbytes.restype = C.c_uint64
        L.tlref_nbytes.argtypes = [_p, C.c_int]
        L.tlref_op.argtypes = [_p, C.c_char_p, _p, C.c_int, _p, C.c_int, _p, C.c_int, C.c_char_p]
        L.tlref_info.argtypes = [_p, C.c_int, _p, _p, _p, _p, _p, _p, _p, _p]
        L.tlref_compute.argtypes = [_p, _p, C.c_int, C.c_int, _p]
        L.tlref_build_flags.restype = C.c_char_p

    def build_flags(self) -> str:
        return self.L.tlref_build_flags().decode()

    def row_size(self, ty: int, ne0: int) -> int:
        return int(self.L.tlref_row_size(ty, ne0))

    def quantize(self, ty: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        rows, n = x.shape
        out = np.zeros((rows, self.row_size(ty, n)), np.uint8)
        self.L.tlref_quantize(ty, _ptr(x), _ptr(out), rows, n)
        return out

    def dequantize(self, ty: int, q: np.ndarray, n: int) -> np.ndarray:
        q = np.ascontiguousarray(q)
        out = np.zeros((q.shape[0], n), np.float32)
        for r in range(q.shape[0]):
            assert self.L.tlref_dequantize(ty, _ptr(q[r]), _ptr(out[r]), n) == 0
        return out

    def act_q8_0(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros((x.shape[0], x.shape[1] // 32 * 34), np.uint8)
        for r in range(x.shape[0]):
            self.L.tlref_act_q8_0(_ptr(x[r]), _ptr(out[r]), x.shape[1])
        return out

    def act_q8_K(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros((x.shape[0], x.shape[1] // 256 * 292), np.uint8)
        for r in range(x.shape[0]):
            self.L.tlref_act_q8_K(_ptr(x[r]), _ptr(out[r]), x.shape[1])
        return out

    def graph(self, mem_bytes: int, n_threads: int = 0) -> "RefGraph":
        return RefGraph(self, mem_bytes, n_threads or (os.cpu_count() or 1))


def ref_gguf_summary(ref: "Ref", path: str) -> str | None:
    """What the reference's own GGUF reader sees in `path` (None when it does not parse, or when the
    reference build predates the hook)."""
    fn = getattr(ref.L, "tlref_gguf_summary", None)
    if fn is None:
        return None
    fn.restype = _i64
    fn.argtypes = [C.c_char_p, C.c_char_p, _i64]
    buf = C.create_string_buffer(1 << 20)
    n = fn(path.encode(), buf, len(buf))
    return None if n < 0 else buf.value.decode()


class RefGraph:
    """A ggml context + op list; tensors are ids. Mirrors the ggml C constructors by name."""

    def __init__(self, ref: Ref, mem_bytes: int, n_threads: int) -> None:
        self.ref = ref
        self.L = ref.L
        self.n_threads = n_threads
        self.h = self.L.tlref_new(mem_bytes, n_threads)
        if not self.h:
            raise MemoryError("ggml_init failed")

    def close(self) -> None:
        if self.h:
            self.L.tlref_free(self.h)
            self.h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    def tensor(self, ty: int, ne, name: str = "", data: np.ndarray | None = None) -> int:
        ne4 = (C.c_int64 * 4)(*(list(ne) + [1] * (4 - len(ne))))
        t = self.L.tlref_tensor(self.h, ty, ne4, name.encode())
        if t < 0:
            raise MemoryError("ggml context is full")
        if data is not None:
            self.write(t, data)
        return t

    def write(self, t: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data)
        n = int(self.L.tlref_nbytes(self.h, t))
        assert data.nbytes == n, (data.nbytes, n)
        C.memmove(self.L.tlref_data(self.h, t), data.ctypes.data, n)

    def write_repeated(self, t: int, data: np.ndarray) -> None:
        """Fills the tensor with `data` repeated end to end (the last copy cut short)."""
        data = np.ascontiguousarray(data)
        n, base = int(self.L.tlref_nbytes(self.h, t)), self.L.tlref_data(self.h, t)
        for off in range(0, n, data.nbytes):
            C.memmove(base + off, data.ctypes.data, min(data.nbytes, n - off))

    def read(self, t: int, dtype=np.float32) -> np.ndarray:
        n = int(self.L.tlref_nbytes(self.h, t))
        buf = np.empty(n, np.uint8)
        C.memmove(buf.ctypes.data, self.L.tlref_data(self.h, t), n)
        return buf.view(dtype)

    def op(self, name: str, srcs=(), ints=(), floats=(), label: str = "") -> int:
        s = (C.c_int * max(1, len(srcs)))(*[(-1 if x is None else x) for x in srcs])
        ia = (C.c_int64 * max(1, len(ints)))(*[int(v) for v in ints])
        fa = (C.c_float * max(1, len(floats)))(*[float(v) for v in floats])
        t = self.L.tlref_op(self.h, name.encode(), s, len(srcs), ia, len(ints), fa, len(floats), label.encode())
        if t < 0:
            raise RuntimeError("tlref_op(%s) failed: %s" % (name, self.L.tlref_error(self.h).decode()))
        return t

    def info(self, t: int) -> dict:
        ty = C.c_int()
        ne = (C.c_int64 * 4)()
        nb = (C.c_uint64 * 4)()
        op = C.create_string_buffer(32)
        params = (C.c_int32 * 16)()
        src = (C.c_int * 10)()
        vs = C.c_int()
        vo = C.c_uint64()
        self.L.tlref_info(self.h, t, C.byref(ty), ne, nb, op, params, src, C.byref(vs), C.byref(vo))
        return dict(ty=ty.value, ne=list(ne), nb=list(nb), op=op.value.decode(), op_params=list(params),
                    src=list(src), view_src=vs.value, view_offs=vo.value)

    def compute(self, outs, repeat: int = 1) -> float:
        """Computes the forward graph of `outs`; returns the best wall time in ms."""
        o = (C.c_int * len(outs))(*outs)
        ms = C.c_double()
        r = self.L.tlref_compute(self.h, o, len(outs), repeat, C.byref(ms))
        if r < 0:
            raise RuntimeError("tlref_compute: " + self.L.tlref_error(self.h).decode())
        return ms.value
