"""Host-side mirror of the reference's native glue (crates/tensorlisp/src/native_cuda.rs:28-168):
``Native`` (device, one weight buffer, the model's state block), ``StateBlock`` (one session's
state) and ``NativeProgram`` (a compiled graph), with the same method names and error behaviour,
forwarding to the C ABI of include/tlb200.h. Nothing here computes; every number comes from the
CUDA library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import TlbError, check
from .graph import F32, I32, I64, INPUT, Graph, TYPE_TRAITS, align256

__all__ = ["EntryCache", "Native", "NativeProgram", "StateBlock", "TlbError", "quantize_rows", "row_size", "to_i32"]

_NP_OF = {0: np.float32, 1: np.float16, 26: np.int32, 27: np.int64, 24: np.int8, 25: np.int16}


def row_size(ty: int, ne0: int) -> int:
    return int(_lib.lib().tlb_row_size(ty, ne0))


class StateBlock:
    """One session's state tensors, laid out like the model's own (native_cuda.rs:29-30)."""

    def __init__(self, handle: C.c_void_p) -> None:
        self.h = handle

    def free(self) -> None:
        if self.h:
            _lib.lib().tlb_buffer_free(self.h)
            self.h = None

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass

    def write(self, offset: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data)
        check(_lib.lib().tlb_buffer_write(self.h, offset, data.ctypes.data_as(C.c_void_p), data.nbytes))

    def read(self, offset: int, nbytes: int) -> np.ndarray:
        out = np.empty(nbytes, np.uint8)
        check(_lib.lib().tlb_buffer_read(self.h, offset, out.ctypes.data_as(C.c_void_p), nbytes))
        return out

    def copy_blocks(self, k_pool_offset: int, v_pool_offset: int, pool_blocks: int, bytes_per_block: int, pairs) -> None:
        """copy_blocks (cuda/paged_attn.rs:434-448): page src -> page dst for every (src, dst), in the K and the V pool."""
        m = np.ascontiguousarray(pairs, np.int64).reshape(-1, 2)
        check(_lib.lib().tlb_state_copy_blocks(self.h, k_pool_offset, v_pool_offset, pool_blocks, bytes_per_block, m.ctypes.data_as(C.c_void_p), len(m)))

    def gather_kv(self, k_pool_offset: int, v_pool_offset: int, pool_blocks: int, kv_heads: int, head_size: int, block_size: int,
                  tables, lens):
        """gather_kv_cache (cuda/paged_attn.rs:450-509): the cached keys and values of the sequences as dense f16 arrays
        [tokens of all sequences, kv_heads, head_size], sequence after sequence."""
        t = np.ascontiguousarray(tables, np.int32)
        n = np.ascontiguousarray(lens, np.int32)
        t = t.reshape(len(n), -1) if len(n) else t.reshape(0, 1)
        total = int(n.sum())
        k = np.zeros((total, kv_heads, head_size), np.float16)
        v = np.zeros((total, kv_heads, head_size), np.float16)
        check(_lib.lib().tlb_state_gather_kv(self.h, k_pool_offset, v_pool_offset, pool_blocks, kv_heads, head_size, block_size,
                                             t.ctypes.data_as(C.c_void_p), t.shape[1], n.ctypes.data_as(C.c_void_p), len(n),
                                             k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))
        return k, v

    def copy_device(self, offset: int, device_ptr: int, nbytes: int) -> None:
        """Device-to-device copy into the buffer (for data that is already in HBM)."""
        check(_lib.lib().tlb_buffer_copy_device(self.h, offset, C.c_void_p(device_ptr), nbytes))

    @property
    def size(self) -> int:
        return int(_lib.lib().tlb_buffer_size(self.h))

    @property
    def device_ptr(self) -> int:
        return int(_lib.lib().tlb_buffer_device_ptr(self.h) or 0)


class Native:
    """Weights, states and the device of one model (native_cuda.rs:32-127)."""

    def __init__(self, ordinal: int = 0) -> None:
        self.L = _lib.lib()
        h = C.c_void_p()
        check(self.L.tlb_device_open(ordinal, C.byref(h)))
        self.dev = h
        self.weights: StateBlock | None = None
        self.weight_loc: list[tuple[int, int]] = []   # weight index -> (buffer index, byte offset)
        self.state: StateBlock | None = None
        self.state_offsets: list[int] = []

    # Native::load (native_cuda.rs:44-82): one buffer, each tensor at a 256-byte aligned offset
    @classmethod
    def load(cls, weights: list[np.ndarray], ordinal: int = 0) -> "Native":
        n = cls(ordinal)
        total = 0
        for w in weights:
            n.weight_loc.append((0, total))
            total += align256(max(int(w.nbytes), 1))
        h = C.c_void_p()
        check(n.L.tlb_weights_create(n.dev, max(total, 1), C.byref(h)))
        n.weights = StateBlock(h)
        for w, (_, off) in zip(weights, n.weight_loc):
            w = np.ascontiguousarray(w)
            check(n.L.tlb_buffer_write(h, off, w.ctypes.data_as(C.c_void_p), w.nbytes))
        return n

    @classmethod
    def load_gguf(cls, path: str, ordinal: int = 0):
        """Model::load_with for the native device (crates/tensorlisp/src/model.rs:458-518 -> native_cuda.rs:44-82): every
        tensor of a GGUF file becomes a weight, in file order, at a 256-byte aligned offset of the one weight buffer, read
        from the file and copied tensor by tensor. Returns (native, file): `file.tensors[i]` describes weight i (name, type,
        shape), `file.program()` is the stored program text; the caller closes both."""
        from .gguf import GgufFile
        f = GgufFile(path)
        n = cls.load([f.tensor_bytes(i) for i in range(len(f.tensors))], ordinal)
        return n, f

    # alloc_states (native_cuda.rs:85-98): one zeroed buffer for all state tensors
    def alloc_states(self, nbytes_per_state: list[int]) -> None:
        total = 0
        self.state_offsets = []
        for b in nbytes_per_state:
            self.state_offsets.append(total)
            total += align256(b)
        self.state = self._zeroed(max(total, 1))

    def _zeroed(self, nbytes: int) -> StateBlock:
        h = C.c_void_p()
        check(self.L.tlb_state_create(self.dev, nbytes, C.byref(h)))
        return StateBlock(h)

    def reset_state(self) -> None:
        check(self.L.tlb_state_zero(self.state.h))

    def new_state_block(self) -> StateBlock:
        return self._zeroed(self.state.size if self.state else 1)

    def fork_block(self, block: StateBlock) -> StateBlock:
        h = C.c_void_p()
        check(self.L.tlb_state_fork(block.h, C.byref(h)))
        return StateBlock(h)

    def reset_block(self, block: StateBlock) -> None:
        check(self.L.tlb_state_zero(block.h))

    def device_name(self) -> str:
        buf = C.create_string_buffer(256)
        check(self.L.tlb_device_name(self.dev, buf, 256))
        return buf.value.decode()

    def sm_count(self) -> int:
        return int(self.L.tlb_device_sm_count(self.dev))

    def stream(self) -> int:
        return int(self.L.tlb_device_stream(self.dev) or 0)

    def sync(self) -> None:
        check(self.L.tlb_device_sync(self.dev))

    def comm_init(self, n_ranks: int, rank: int, unique_id: bytes | None) -> None:
        buf = C.create_string_buffer(unique_id, 128) if unique_id is not None else None
        check(self.L.tlb_comm_init(self.dev, n_ranks, rank, buf))

    def comm_p2p_export(self) -> bytes:
        """This rank's exchange buffer for the peer-memory all-reduce, as a 64-byte CUDA IPC handle."""
        buf = C.create_string_buffer(64)
        check(self.L.tlb_comm_p2p_export(self.dev, buf))
        return buf.raw

    def comm_p2p_import(self, handles: list[bytes]) -> None:
        """Handles of all ranks, in rank order (as gathered by the host's own channel)."""
        blob = b"".join(handles)
        check(self.L.tlb_comm_p2p_import(self.dev, C.create_string_buffer(blob, len(blob))))

    @staticmethod
    def comm_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(_lib.lib().tlb_comm_unique_id(buf))
        return buf.raw

    def close(self) -> None:
        for b in (self.weights, self.state):
            if b:
                b.free()
        self.weights = self.state = None
        if self.dev:
            self.L.tlb_device_close(self.dev)
            self.dev = None


class NativeProgram:
    """A compiled graph with what is needed to feed and read it (native_cuda.rs:129-168)."""

    def __init__(self, native: Native, handle: C.c_void_p, graph: Graph, outputs: list[tuple[str, int]]) -> None:
        self.native = native
        self.h = handle
        self.graph = graph
        self._outputs = outputs

    @classmethod
    def compile(cls, native: Native, graph: Graph, outputs: list[tuple[str, int]] | None = None) -> "NativeProgram":
        outputs = outputs if outputs is not None else [(graph.tensors[t].name, t) for t in graph.keep]
        for _, t in outputs:
            if t not in graph.keep:
                graph.keep.append(t)
        g, keep = graph.to_c()
        nw, ns = len(native.weight_loc), len(native.state_offsets)
        wb = (C.c_uint32 * max(nw, 1))(*[b for b, _ in native.weight_loc])
        wo = (C.c_uint64 * max(nw, 1))(*[o for _, o in native.weight_loc])
        so = (C.c_uint64 * max(ns, 1))(*native.state_offsets)
        leaves = _lib.tlb_leaves(wb, wo, nw, so, ns)
        h = C.c_void_p()
        err = C.create_string_buffer(4096)
        st = native.L.tlb_program_compile(native.dev, C.byref(g), C.byref(leaves), C.byref(h), err, 4096)
        del keep
        if st != 0:
            raise TlbError(st, err.value.decode(errors="replace"))
        return cls(native, h, graph, outputs)

    def set_input(self, i: int, data: np.ndarray | bytes) -> None:
        if isinstance(data, (bytes, bytearray)):
            data = np.frombuffer(data, np.uint8)
        data = np.ascontiguousarray(data)
        check(self.native.L.tlb_program_set_input(self.h, i, data.ctypes.data_as(C.c_void_p), data.nbytes))

    def _buffers(self, state: StateBlock | None):
        st = state if state is not None else self.native.state
        w = self.native.weights
        arr = (C.c_void_p * 1)(w.h if w else None)
        return arr, (1 if w else 0), (st.h if st else None)

    def feed_input(self, i: int, tensor: int) -> None:
        """The bytes of a kept arena tensor become input i of the next run (device-side copy, enqueued)."""
        check(self.native.L.tlb_program_feed_input(self.h, i, tensor))

    def run(self, state: StateBlock | None = None) -> None:
        arr, n, st = self._buffers(state)
        check(self.native.L.tlb_program_run(self.h, arr, n, st))

    def enqueue(self, state: StateBlock | None = None) -> None:
        arr, n, st = self._buffers(state)
        check(self.native.L.tlb_program_enqueue(self.h, arr, n, st))

    def profile(self, state: StateBlock | None = None) -> list[tuple[str, float]]:
        """Runs once launch by launch; returns (label, device milliseconds) per launch."""
        arr, n, st = self._buffers(state)
        k = self.dispatch_count()
        ms = (C.c_float * max(k, 1))()
        check(self.native.L.tlb_program_profile(self.h, arr, n, st, ms, k))
        return list(zip(self.labels(), [float(v) for v in ms[:k]]))

    def read(self, tensor: int, dtype=None) -> np.ndarray:
        """The tensor's bytes as an array of its own element type, in ndarray (outermost first) order."""
        T = self.graph.tensors[tensor]
        n = T.nbytes()
        out = np.empty(n, np.uint8)
        check(self.native.L.tlb_program_read(self.h, tensor, n, out.ctypes.data_as(C.c_void_p)))
        dt = dtype or _NP_OF.get(T.ty)
        if dt is None:
            return out
        shape = [d for d in reversed(T.ne)]
        while len(shape) > 1 and shape[0] == 1:
            shape.pop(0)
        return out.view(dt).reshape(shape)

    def outputs(self) -> list[tuple[str, np.ndarray]]:
        return [(name, self.read(t)) for name, t in self._outputs]

    def dispatch_count(self) -> int:
        return int(self.native.L.tlb_program_dispatch_count(self.h))

    def kernel_count(self) -> int:
        """Kernel launches per run (those of the CUDA graph captured last; 0 before the first run)."""
        return int(self.native.L.tlb_program_kernel_count(self.h))

    def labels(self) -> list[str]:
        return [self.native.L.tlb_program_label(self.h, i).decode() for i in range(self.dispatch_count())]

    def tensor_ptr(self, tensor: int) -> tuple[int, int]:
        n = C.c_uint64()
        p = self.native.L.tlb_program_tensor_ptr(self.h, tensor, C.byref(n))
        return int(p or 0), int(n.value)

    def arena_bytes(self) -> int:
        return int(self.native.L.tlb_program_arena_bytes(self.h))

    def free(self) -> None:
        if self.h:
            self.native.L.tlb_program_free(self.h)
            self.h = None

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass


def to_i32(name: str, values: np.ndarray) -> np.ndarray:
    """An i32 input arrives as whole-number f32 values (crates/tensorlisp/src/model.rs:940-952); anything else is an
    input error that names the input and the value."""
    v = np.ascontiguousarray(values)
    if v.dtype.kind in "iu":
        return v.astype(np.int32)
    f = v.astype(np.float32).reshape(-1)
    bad = ~((f == np.trunc(f)) & (f >= np.float32(-2 ** 31)) & (f <= np.float32(2 ** 31 - 1)))     # NaN compares false
    if bad.any():
        raise ValueError("input %r is i32 but contains %s" % (name, f[np.argmax(bad)]))
    return f.astype(np.int64).clip(-2 ** 31, 2 ** 31 - 1).astype(np.int32).reshape(v.shape)


class EntryCache:
    """Inner::run_native (crates/tensorlisp/src/model.rs:1038-1093): the programs of a model's entries, compiled per
    combination of input shapes when first seen and replayed afterwards. An entry keeps at most eight programs; a ninth
    shape drops the oldest (and frees it). `build(name, shapes)` returns the entry's Graph for those input shapes with
    its outputs marked (the reference builds it by running the Scheme program); `compile` is NativeProgram.compile unless
    a test passes its own."""

    LIMIT = 8

    def __init__(self, native, build, compile=None) -> None:
        self.native, self.build = native, build
        self.compile = compile or (lambda native, graph: NativeProgram.compile(native, graph))
        self.programs: dict[str, list[tuple[tuple, object]]] = {}

    def program(self, name: str, shapes: tuple):
        lst = self.programs.setdefault(name, [])
        for key, prog in lst:
            if key == shapes:
                return prog
        prog = self.compile(self.native, self.build(name, shapes))
        if len(lst) >= self.LIMIT:
            _, oldest = lst.pop(0)
            oldest.free()
        lst.append((shapes, prog))
        return prog

    def run(self, name: str, inputs, state: StateBlock | None = None):
        """inputs: arrays in the entry's input order. f32 goes in as it is; an input the graph declares i32 takes
        whole-number values. Returns the outputs as (name, array) pairs."""
        arrays = [np.asarray(a) for a in inputs]
        prog = self.program(name, tuple(tuple(a.shape) for a in arrays))
        declared = [t for t in prog.graph.tensors if t.storage_kind == INPUT]
        declared.sort(key=lambda t: t.storage_index)
        for i, a in enumerate(arrays):
            t = declared[i] if i < len(declared) else None
            if t is not None and t.ty in (I32, I64):
                a = to_i32(t.name, a) if t.ty == I32 else to_i32(t.name, a).astype(np.int64)
            elif t is not None and t.ty == F32:
                a = np.ascontiguousarray(a, np.float32)
            prog.set_input(i, a)
        prog.run(state)
        return prog.outputs()

    def free(self) -> None:
        for lst in self.programs.values():
            for _, prog in lst:
                prog.free()
        self.programs = {}


def quantize_rows(native: Native, ty: int, x: np.ndarray) -> np.ndarray:
    """DType::from_f32 (crates/tensorlisp/src/dtype.rs:98-124): f32 [rows, n] -> blocks [rows, row bytes]."""
    x = np.ascontiguousarray(x, np.float32)
    rows, n = x.shape
    name, blck, size = TYPE_TRAITS.get(ty, ("?", 1, 0))      # an unknown type is refused by name by the library
    out = np.zeros((rows, size * n // blck if n % blck == 0 else 0), np.uint8)
    check(native.L.tlb_quantize_rows(native.dev, ty, x.ctypes.data_as(C.c_void_p), rows, n,
                                     out.ctypes.data_as(C.c_void_p)))
    return out
