"""Builds the graph IR the executor compiles (include/tlb200.h: tlb_tensor / tlb_graph).

In the reference a Scheme program calls generated ``(ggml-<op> ...)`` wrappers of the ggml C API
(README.md:120-123) and crates/tensorlisp/src/native_ir.rs:30-114 copies the resulting cgraph into
the IR field by field. Neither Scheme nor Rust exists on the machines this runs on, so this module
restates the shape / stride / op_params rules of the ggml constructors it needs
(vendor/ggml/src/ggml.c; each method names its constructor). tests/test_graph_ir.py checks every
one against ggml itself through the reference build.

Tensor ids are indices into ``Graph.tensors``; ``nodes`` are appended in call order, which is the
order ggml_build_forward_expand visits a program written top to bottom.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np
from dataclasses import dataclass, field

from . import _lib

F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 = 0, 1, 2, 3, 6, 7, 8
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
I8, I16, I32, I64, BF16 = 24, 25, 26, 27, 30

# (name, elements per block, bytes per block): crates/kernels/src/graph.rs:30-50
TYPE_TRAITS = {
    F32: ("f32", 1, 4), F16: ("f16", 1, 2), Q4_0: ("q4_0", 32, 18), Q4_1: ("q4_1", 32, 20),
    Q5_0: ("q5_0", 32, 22), Q5_1: ("q5_1", 32, 24), Q8_0: ("q8_0", 32, 34), Q2_K: ("q2_K", 256, 84),
    Q3_K: ("q3_K", 256, 110), Q4_K: ("q4_K", 256, 144), Q5_K: ("q5_K", 256, 176), Q6_K: ("q6_K", 256, 210),
    I8: ("i8", 1, 1), I16: ("i16", 1, 2), I32: ("i32", 1, 4), I64: ("i64", 1, 8), BF16: ("bf16", 1, 2),
}

WEIGHT, STATE, INPUT, TEMP = 0, 1, 2, 3

UNARY_OPS = {"abs": 0, "sgn": 1, "neg": 2, "step": 3, "tanh": 4, "elu": 5, "relu": 6, "sigmoid": 7, "gelu": 8,
             "gelu_quick": 9, "silu": 10, "hardswish": 11, "hardsigmoid": 12, "exp": 13, "expm1": 14,
             "softplus": 15, "gelu_erf": 16, "xielu": 17, "floor": 18, "ceil": 19, "round": 20, "trunc": 21}
GLU_OPS = {"reglu": 0, "geglu": 1, "swiglu": 2, "swiglu_oai": 3, "geglu_erf": 4, "geglu_quick": 5}


def f32_bits(x: float) -> int:
    return struct.unpack("<i", struct.pack("<f", float(x)))[0]


def row_size(ty: int, ne0: int) -> int:
    _, blck, size = TYPE_TRAITS[ty]
    assert ne0 % blck == 0, "row of %d elements is not a multiple of the block size %d" % (ne0, blck)
    return size * ne0 // blck


def align256(n: int) -> int:
    return (n + 255) // 256 * 256


@dataclass
class Tensor:
    ty: int
    ne: list
    nb: list
    op: str = "NONE"
    op_params: list = field(default_factory=lambda: [0] * 16)
    src: list = field(default_factory=lambda: [-1] * 10)
    view_src: int = -1
    view_offs: int = 0
    storage_kind: int = TEMP
    storage_index: int = 0
    name: str = ""

    def nelements(self) -> int:
        return self.ne[0] * self.ne[1] * self.ne[2] * self.ne[3]

    def nbytes(self) -> int:  # ggml_nbytes
        if 0 in self.ne:
            return 0
        _, blck, size = TYPE_TRAITS[self.ty]
        n = size + (self.ne[0] - 1) * self.nb[0] if blck == 1 else self.ne[0] * self.nb[0] // blck
        for i in range(1, 4):
            n += (self.ne[i] - 1) * self.nb[i]
        return n


class Graph:
    """An op list in ggml's vocabulary; every method returns the id of the new tensor."""

    def __init__(self) -> None:
        self.tensors: list[Tensor] = []
        self.nodes: list[int] = []
        self.keep: list[int] = []
        self.n_weights = 0
        self.n_states = 0
        self.n_inputs = 0

    # ------------------------------------------------------------------ leaves
    def _new(self, ty: int, ne, view_src: int = -1, view_offs: int = 0, name: str = "") -> int:
        # ggml_new_tensor_impl (ggml.c:1690-1767): a view of a view resolves to the root
        ne = list(ne) + [1] * (4 - len(ne))
        if view_src >= 0 and self.tensors[view_src].view_src >= 0:
            view_offs += self.tensors[view_src].view_offs
            view_src = self.tensors[view_src].view_src
        _, blck, size = TYPE_TRAITS[ty]
        nb = [size, size * (ne[0] // blck), 0, 0]
        nb[2] = nb[1] * ne[1]
        nb[3] = nb[2] * ne[2]
        self.tensors.append(Tensor(ty, ne, nb, view_src=view_src, view_offs=view_offs, name=name))
        return len(self.tensors) - 1

    def weight(self, ty: int, ne, name: str = "") -> int:
        t = self._new(ty, ne, name=name)
        self.tensors[t].storage_kind, self.tensors[t].storage_index = WEIGHT, self.n_weights
        self.n_weights += 1
        return t

    def state(self, ty: int, ne, name: str = "") -> int:
        t = self._new(ty, ne, name=name)
        self.tensors[t].storage_kind, self.tensors[t].storage_index = STATE, self.n_states
        self.n_states += 1
        return t

    def input(self, ty: int, ne, name: str = "") -> int:
        t = self._new(ty, ne, name=name)
        self.tensors[t].storage_kind, self.tensors[t].storage_index = INPUT, self.n_inputs
        self.n_inputs += 1
        return t

    def output(self, t: int) -> int:
        self.keep.append(t)
        return t

    def set_name(self, t: int, name: str) -> int:
        self.tensors[t].name = name
        return t

    # ------------------------------------------------------------------ helpers
    def _node(self, t: int, op: str, srcs=(), params=None, name: str = "") -> int:
        T = self.tensors[t]
        T.op = op
        for i, s in enumerate(srcs):
            T.src[i] = -1 if s is None else s
        if params:
            for i, v in params.items():
                T.op_params[i] = v
        if name:
            T.name = name
        elif not T.name:
            T.name = "%s_%d" % (op.lower(), t)
        self.nodes.append(t)
        return t

    def _dup(self, a: int) -> int:  # ggml_dup_tensor
        A = self.tensors[a]
        return self._new(A.ty, A.ne)

    def _view(self, a: int) -> int:  # ggml_view_tensor: same shape and strides, aliases a
        A = self.tensors[a]
        t = self._new(A.ty, A.ne, view_src=a, view_offs=0)
        self.tensors[t].nb = list(A.nb)
        return t

    # ------------------------------------------------------------------ ops
    def mul_mat(self, a: int, b: int, name: str = "") -> int:  # ggml_mul_mat (ggml.c:3221-3241)
        A, B = self.tensors[a], self.tensors[b]
        assert A.ne[0] == B.ne[0] and B.ne[2] % A.ne[2] == 0 and B.ne[3] % A.ne[3] == 0, "ggml_can_mul_mat"
        t = self._new(F32, [A.ne[1], B.ne[1], B.ne[2], B.ne[3]])
        return self._node(t, "MUL_MAT", [a, b], name=name)

    def _bin(self, op: str, a: int, b: int, name: str) -> int:
        return self._node(self._dup(a), op, [a, b], name=name)

    def add(self, a, b, name=""):
        return self._bin("ADD", a, b, name)

    def sub(self, a, b, name=""):
        return self._bin("SUB", a, b, name)

    def mul(self, a, b, name=""):
        return self._bin("MUL", a, b, name)

    def div(self, a, b, name=""):
        return self._bin("DIV", a, b, name)

    def rms_norm(self, a: int, eps: float, name: str = "") -> int:  # ggml_rms_norm (ggml.c:3162)
        return self._node(self._dup(a), "RMS_NORM", [a], {0: f32_bits(eps)}, name)

    def norm(self, a: int, eps: float, name: str = "") -> int:
        return self._node(self._dup(a), "NORM", [a], {0: f32_bits(eps)}, name)

    def unary(self, a: int, op, name: str = "") -> int:  # ggml_unary
        code = UNARY_OPS[op] if isinstance(op, str) else int(op)
        return self._node(self._dup(a), "UNARY", [a], {0: code}, name)

    def silu(self, a: int, name: str = "") -> int:
        return self.unary(a, "silu", name)

    def glu(self, a: int, op="swiglu", swapped: bool = False, b: int | None = None, name: str = "") -> int:
        # ggml_glu_impl (ggml.c:2905-2930)
        code = GLU_OPS[op] if isinstance(op, str) else int(op)
        A = self.tensors[a]
        ne = list(A.ne)
        if b is None:
            ne[0] //= 2
        t = self._new(A.ty, ne)
        return self._node(t, "GLU", [a, b], {0: code, 1: int(swapped)}, name)

    def scale(self, a: int, s: float, bias: float = 0.0, name: str = "") -> int:  # ggml_scale_impl (ggml.c:3395)
        return self._node(self._dup(a), "SCALE", [a], {0: f32_bits(s), 1: f32_bits(bias)}, name)

    def sqr(self, a, name=""):
        return self._node(self._dup(a), "SQR", [a], name=name)

    def sqrt(self, a, name=""):
        return self._node(self._dup(a), "SQRT", [a], name=name)

    def sin(self, a, name=""):
        return self._node(self._dup(a), "SIN", [a], name=name)

    def cos(self, a, name=""):
        return self._node(self._dup(a), "COS", [a], name=name)

    def log(self, a, name=""):
        return self._node(self._dup(a), "LOG", [a], name=name)

    def leaky_relu(self, a, negative_slope: float, name=""):  # ggml_leaky_relu (not in place)
        return self._node(self._dup(a), "LEAKY_RELU", [a], {0: f32_bits(negative_slope)}, name)

    def fill(self, a, c: float, name=""):  # ggml_fill (ggml.c:5294-5317): a tensor shaped like a, every element c
        return self._node(self._dup(a), "FILL", [a], {0: f32_bits(c)}, name)

    def clamp(self, a, lo: float, hi: float, name=""):
        # ggml_clamp is in place: the result is a view of a
        return self._node(self._view(a), "CLAMP", [a], {0: f32_bits(lo), 1: f32_bits(hi)}, name)

    def rope_ext(self, a: int, pos: int, ff: int | None, n_dims: int, mode: int, n_ctx_orig: int, freq_base: float,
                 freq_scale: float, ext_factor: float, attn_factor: float, beta_fast: float, beta_slow: float,
                 name: str = "") -> int:
        # ggml_rope_impl (ggml.c:4169-4225)
        params = {0: 0, 1: n_dims, 2: mode, 3: 0, 4: n_ctx_orig, 5: f32_bits(freq_base), 6: f32_bits(freq_scale),
                  7: f32_bits(ext_factor), 8: f32_bits(attn_factor), 9: f32_bits(beta_fast), 10: f32_bits(beta_slow)}
        return self._node(self._dup(a), "ROPE", [a, pos, ff], params, name)

    def soft_max_ext(self, a: int, mask: int | None, scale: float, max_bias: float = 0.0, name: str = "") -> int:
        # ggml_soft_max_impl (ggml.c:4054-4076)
        return self._node(self._dup(a), "SOFT_MAX", [a, mask], {0: f32_bits(scale), 1: f32_bits(max_bias)}, name)

    def get_rows(self, a: int, b: int, name: str = "") -> int:  # ggml_get_rows (ggml.c:3895-3909)
        A, B = self.tensors[a], self.tensors[b]
        ty = I32 if A.ty == I32 else F32
        t = self._new(ty, [A.ne[0], B.ne[0], B.ne[1], B.ne[2]])
        return self._node(t, "GET_ROWS", [a, b], name=name)

    def set_rows(self, a: int, b: int, c: int, name: str = "") -> int:  # ggml_set_rows (ggml.c:3942-3959)
        # the node is a view of the destination a; sources are the rows b, the ids c, and a itself
        return self._node(self._view(a), "SET_ROWS", [b, c, a], name=name)

    def cpy(self, a: int, b: int, name: str = "") -> int:  # ggml_cpy_impl (ggml.c:3527-3547): a view of b
        t = self._view(b)
        if not name:
            name = (self.tensors[b].name + " (copy of %s)" % self.tensors[a].name) if self.tensors[b].name else \
                " (copy of %s)" % self.tensors[a].name
        return self._node(t, "CPY", [a, b], name=name[:63])

    def cast(self, a: int, ty: int, name: str = "") -> int:  # ggml_cast (ggml.c:3549-3563): src[1] is itself
        A = self.tensors[a]
        t = self._new(ty, A.ne)
        return self._node(t, "CPY", [a, t], name=name or (A.name + " (copy)")[:63])

    def cont(self, a: int, name: str = "") -> int:  # ggml_cont_impl
        return self._node(self._dup(a), "CONT", [a], name=name or (self.tensors[a].name + " (cont)")[:63])

    def reshape(self, a: int, ne, name: str = "") -> int:  # ggml_reshape_4d
        A = self.tensors[a]
        ne = list(ne) + [1] * (4 - len(ne))
        assert ne[0] * ne[1] * ne[2] * ne[3] == A.nelements(), "reshape changes the element count"
        t = self._new(A.ty, ne, view_src=a, view_offs=0)
        return self._node(t, "RESHAPE", [a], name=name or (A.name + " (reshaped)")[:63])

    def view(self, a: int, ne, nb1: int = 0, nb2: int = 0, nb3: int = 0, offset: int = 0, name: str = "") -> int:
        # ggml_view_impl + ggml_view_{1..4}d (ggml.c:3700-3800)
        A = self.tensors[a]
        nd = len(ne)
        ne = list(ne) + [1] * (4 - len(ne))
        t = self._new(A.ty, ne, view_src=a, view_offs=offset)
        T = self.tensors[t]
        if nd == 2:
            T.nb[1] = nb1
            T.nb[2] = T.nb[1] * ne[1]
            T.nb[3] = T.nb[2]
        elif nd == 3:
            T.nb[1], T.nb[2] = nb1, nb2
            T.nb[3] = T.nb[2] * ne[2]
        elif nd == 4:
            T.nb[1], T.nb[2], T.nb[3] = nb1, nb2, nb3
        params = {0: offset & 0xffffffff, 1: (offset >> 32) & 0xffffffff}
        params = {k: (v - (1 << 32) if v >= (1 << 31) else v) for k, v in params.items()}
        return self._node(t, "VIEW", [a], params, name or (A.name + " (view)")[:63])

    def permute(self, a: int, ax0: int, ax1: int, ax2: int, ax3: int, name: str = "") -> int:  # ggml_permute
        A = self.tensors[a]
        t = self._view(a)
        T = self.tensors[t]
        ne, nb = [0] * 4, [0] * 4
        for i, ax in enumerate((ax0, ax1, ax2, ax3)):
            ne[ax], nb[ax] = A.ne[i], A.nb[i]
        T.ne, T.nb = ne, nb
        return self._node(t, "PERMUTE", [a], {0: ax0, 1: ax1, 2: ax2, 3: ax3}, name or (A.name + " (permuted)")[:63])

    def transpose(self, a: int, name: str = "") -> int:  # ggml_transpose
        A = self.tensors[a]
        t = self._view(a)
        T = self.tensors[t]
        T.ne = [A.ne[1], A.ne[0], A.ne[2], A.ne[3]]
        T.nb = [A.nb[1], A.nb[0], A.nb[2], A.nb[3]]
        return self._node(t, "TRANSPOSE", [a], name=name or (A.name + " (transposed)")[:63])

    def flash_attn_ext(self, q, k, v, mask, scale: float, max_bias: float = 0.0, softcap: float = 0.0, name="") -> int:
        # ggml_flash_attn_ext (ggml.c:5402-5444): result is permuted [Dv, heads, queries, batch]
        Q, V = self.tensors[q], self.tensors[v]
        t = self._new(F32, [V.ne[0], Q.ne[2], Q.ne[1], Q.ne[3]])
        return self._node(t, "FLASH_ATTN_EXT", [q, k, v, mask],
                          {0: f32_bits(scale), 1: f32_bits(max_bias), 2: f32_bits(softcap)}, name)

    def argmax(self, a: int, name: str = "") -> int:  # ggml_argmax (ggml.c:2539-2545)
        t = self._new(I32, [self.tensors[a].ne[1]])
        return self._node(t, "ARGMAX", [a], name=name)

    def concat(self, a: int, b: int, dim: int, name: str = "") -> int:
        A, B = self.tensors[a], self.tensors[b]
        ne = list(A.ne)
        ne[dim] += B.ne[dim]
        return self._node(self._new(A.ty, ne), "CONCAT", [a, b], {0: dim}, name)

    def repeat(self, a: int, like: int, name: str = "") -> int:
        A, B = self.tensors[a], self.tensors[like]
        return self._node(self._new(A.ty, B.ne), "REPEAT", [a], name=name)

    def sum_rows(self, a: int, name: str = "") -> int:
        A = self.tensors[a]
        return self._node(self._new(A.ty, [1, A.ne[1], A.ne[2], A.ne[3]]), "SUM_ROWS", [a], name=name)

    def mean(self, a: int, name: str = "") -> int:  # ggml_mean (ggml.c:2522-2532): f32 whatever the source type
        A = self.tensors[a]
        return self._node(self._new(F32, [1, A.ne[1], A.ne[2], A.ne[3]]), "MEAN", [a], name=name)

    def arange(self, start: float, stop: float, step: float, name: str = "") -> int:  # ggml_arange (ggml.c:5380-5398)
        import math
        assert stop > start
        # the count is taken in f32, as ggml takes it
        steps = int(math.ceil(float(np.float32(np.float32(stop) - np.float32(start)) / np.float32(step))))
        return self._node(self._new(F32, [steps]), "ARANGE", [], {0: f32_bits(start), 1: f32_bits(stop), 2: f32_bits(step)}, name)

    # ------------------------------------------------------------------ image ops (shape rules of ggml.c)
    @staticmethod
    def _conv_out(ins: int, ks: int, s: int, p: int, d: int) -> int:  # ggml_calc_conv_output_size (ggml.c:4444-4446)
        return (ins + 2 * p - d * (ks - 1) - 1) // s + 1

    def im2col(self, kernel: int, data: int, s0: int, s1: int, p0: int, p1: int, d0: int, d1: int, is_2d: bool,
               dst_type: int = F32, name: str = "") -> int:  # ggml_im2col (ggml.c:4452-4494)
        A, B = self.tensors[kernel], self.tensors[data]
        if is_2d:
            assert A.ne[2] == B.ne[2]
        else:
            assert B.ne[1] == A.ne[1] and B.ne[3] == 1
        oh = self._conv_out(B.ne[1], A.ne[1], s1, p1, d1) if is_2d else 0
        ow = self._conv_out(B.ne[0], A.ne[0], s0, p0, d0)
        assert ow > 0 and (not is_2d or oh > 0), "data too small for the kernel"
        ne = [A.ne[2] * A.ne[1] * A.ne[0] if is_2d else A.ne[1] * A.ne[0], ow, oh if is_2d else B.ne[2], B.ne[3] if is_2d else 1]
        return self._node(self._new(dst_type, ne), "IM2COL", [kernel, data],
                          {0: s0, 1: s1, 2: p0, 3: p1, 4: d0, 5: d1, 6: 1 if is_2d else 0}, name)

    def interpolate(self, a: int, ne0: int, ne1: int, ne2: int, ne3: int, mode: int, name: str = "") -> int:
        """ggml_interpolate (ggml.c:5061-5082): mode = 0 nearest / 1 bilinear / 2 bicubic, | 1<<8 align corners, | 1<<9 antialias."""
        A = self.tensors[a]
        assert (mode & 0xFF) < 3 and A.ty == F32
        assert not (mode & (1 << 9)) or (mode & 0xFF) == 1, "antialias is bilinear only"
        return self._node(self._new(A.ty, [ne0, ne1, ne2, ne3]), "UPSCALE", [a], {0: mode}, name)

    def upscale(self, a: int, scale_factor: int, mode: int = 0, name: str = "") -> int:  # ggml_upscale (ggml.c:5084-5091)
        A = self.tensors[a]
        assert scale_factor > 1
        return self.interpolate(a, A.ne[0] * scale_factor, A.ne[1] * scale_factor, A.ne[2], A.ne[3], mode, name)

    def pool_2d(self, a: int, op: int, k0: int, k1: int, s0: int, s1: int, p0: float, p1: float, name: str = "") -> int:
        """ggml_pool_2d (ggml.c:4970-4972, 5004-5033): op 0 = max, 1 = average; the output size is computed in f32."""
        A = self.tensors[a]
        out = lambda ins, ks, s, p: int((np.float32(ins) + np.float32(2) * np.float32(p) - np.float32(ks)) / np.float32(s) + np.float32(1))
        ne = [out(A.ne[0], k0, s0, p0), out(A.ne[1], k1, s1, p1), A.ne[2], A.ne[3]]
        assert ne[0] > 0 and ne[1] > 0
        return self._node(self._new(F32, ne), "POOL_2D", [a], {0: op, 1: k0, 2: k1, 3: s0, 4: s1, 5: int(p0), 6: int(p1)}, name)

    def conv_2d_dw(self, kernel: int, data: int, s0: int, s1: int, p0: int, p1: int, d0: int, d1: int, name: str = "") -> int:
        """ggml_conv_2d_dw_direct (ggml.c:4812-4848) on WHCN data (contiguous rows)."""
        A, B = self.tensors[kernel], self.tensors[data]
        assert A.ne[2] == 1 and A.ne[3] == B.ne[2]
        assert not (B.nb[0] > B.nb[2] and B.nb[1] > B.nb[0] and B.nb[2] == TYPE_TRAITS[B.ty][2]), "channel-contiguous data is not modelled here"
        ne = [self._conv_out(B.ne[0], A.ne[0], s0, p0, d0), self._conv_out(B.ne[1], A.ne[1], s1, p1, d1), B.ne[2], B.ne[3]]
        return self._node(self._new(B.ty, ne), "CONV_2D_DW", [kernel, data], {0: s0, 1: s1, 2: p0, 3: p1, 4: d0, 5: d1}, name)

    def pad_ext(self, a: int, lp0: int, rp0: int, lp1: int, rp1: int, lp2: int, rp2: int, lp3: int, rp3: int, name: str = "") -> int:
        A = self.tensors[a]   # ggml_pad_ext (ggml.c:5139-5172)
        ne = [A.ne[0] + lp0 + rp0, A.ne[1] + lp1 + rp1, A.ne[2] + lp2 + rp2, A.ne[3] + lp3 + rp3]
        return self._node(self._new(A.ty, ne), "PAD", [a], {0: lp0, 1: rp0, 2: lp1, 3: rp1, 4: lp2, 5: rp2, 6: lp3, 7: rp3, 8: 0}, name)

    def pad(self, a: int, p0: int, p1: int, p2: int, p3: int, name: str = "") -> int:  # ggml_pad: right padding only
        return self.pad_ext(a, 0, p0, 0, p1, 0, p2, 0, p3, name)

    def pad_reflect_1d(self, a: int, p0: int, p1: int, name: str = "") -> int:  # ggml_pad_reflect_1d (ggml.c:5195-5222)
        A = self.tensors[a]
        assert 0 <= p0 < A.ne[0] and 0 <= p1 < A.ne[0] and A.ty == F32
        assert A.nb[0] == 4 and all(A.nb[i] == A.nb[i - 1] * A.ne[i - 1] for i in (1, 2, 3)), "contiguous input only"
        return self._node(self._new(A.ty, [A.ne[0] + p0 + p1, A.ne[1], A.ne[2], A.ne[3]]), "PAD_REFLECT_1D", [a], {0: p0, 1: p1}, name)

    def cumsum(self, a: int, name: str = "") -> int:
        return self._node(self._dup(a), "CUMSUM", [a], name=name)

    # the paged nodes of scheme/core.ss:222-271
    @staticmethod
    def paged_userdata(kind: int, kv_heads: int, block_size: int, max_context: int, scale: float) -> int:
        assert 0 < kv_heads < 16, "kv-heads must be 1..15"
        assert block_size in (8, 16, 32), "block-size must be 8, 16 or 32"
        assert 0 < max_context < 65536, "max-context must be 1..65535"
        return kind + kv_heads * 16 + block_size * 256 + max_context * 65536 + ((f32_bits(scale) & 0xffffffff) << 32)

    def _custom(self, ty: int, ne, srcs, userdata: int, name: str) -> int:
        # ggml_custom_4d (ggml.c:6087-6104): params = {fun ptr (NULL), n_tasks (1), userdata}
        t = self._new(ty, ne)
        lo, hi = userdata & 0xffffffff, (userdata >> 32) & 0xffffffff
        sg = lambda v: v - (1 << 32) if v >= (1 << 31) else v
        return self._node(t, "CUSTOM", list(srcs), {2: 1, 4: sg(lo), 5: sg(hi)}, name)

    def paged_attention(self, q, kc, vc, tables, lens, block_size: int, max_context: int, scale: float,
                        kv_heads: int = 1, name: str = "") -> int:
        Q = self.tensors[q]
        ud = self.paged_userdata(1, kv_heads, block_size, max_context, scale)
        return self._custom(F16, [Q.ne[0], Q.ne[1], Q.ne[2], 1], [q, kc, vc, tables, lens], ud, name or "paged_attention")

    def paged_cache_write(self, k, v, kc, vc, slots, block_size: int, kv_heads: int = 1, name: str = "") -> int:
        ud = self.paged_userdata(2, kv_heads, block_size, 1, 1.0)
        return self._custom(F16, [1, 1, 1, 1], [k, v, kc, vc, slots], ud, name or "paged_cache_write")

    # tensor-parallel pseudo-op (no ggml counterpart): in-place sum over the ranks of a communicator
    def allreduce(self, a: int, name: str = "") -> int:
        return self._node(self._view(a), "ALLREDUCE", [a], name=name or "allreduce")

    # ------------------------------------------------------------------ C structs
    def to_c(self):
        """(tlb_graph, keepalive) for tlb_program_compile."""
        n = len(self.tensors)
        arr = (_lib.tlb_tensor * max(n, 1))()
        for i, t in enumerate(self.tensors):
            c = arr[i]
            c.ty = t.ty
            for k in range(4):
                c.ne[k] = t.ne[k]
                c.nb[k] = t.nb[k]
            c.op = t.op.encode()[:31]
            for k in range(16):
                c.op_params[k] = t.op_params[k]
            for k in range(10):
                c.src[k] = t.src[k]
            c.view_src = t.view_src
            c.view_offs = t.view_offs
            c.storage_kind = t.storage_kind
            c.storage_index = t.storage_index
            c.name = t.name.encode()[:63]
        nodes = (C.c_int32 * max(len(self.nodes), 1))(*self.nodes)
        keep = (C.c_int32 * max(len(self.keep), 1))(*self.keep)
        g = _lib.tlb_graph(arr, n, nodes, len(self.nodes), keep, len(self.keep))
        return g, (arr, nodes, keep)
