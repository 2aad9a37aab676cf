"""GGUF (version 3) files as tensorlisp uses them (reference: crates/tensorlisp/src/gguf.rs:87-489 over the
vendored gguf.cpp; program keys crates/tensorlisp/src/program.rs:3-15): a reader that maps tensors without
copying, a writer, the TL_VER / TL_TXT / TL_ASSET.<name> keys, and `quantize_file`, the `tl quantize`
counterpart that quantizes weights on the GPU with the library's bit-exact row quantizers
(crates/tensorlisp/src/quantize.rs:193-267: only 2-D tensors whose rows are a whole number of blocks).

The container format is the published GGUF layout: magic "GGUF", u32 version, u64 tensor count, u64 key
count, keys (string, u32 type, value), tensor infos (string name, u32 rank, u64 dims, u32 ggml type, u64
offset into the data section), padding to `general.alignment` (32 by default), tensor data each aligned
to it. Strings are u64 length + bytes; arrays are u32 element type + u64 count + elements.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

from .graph import row_size

MAGIC = 0x46554747
TL_VER, TL_TXT, TL_BIN, TL_ASSET_PREFIX = "TL_VER", "TL_TXT", "TL_BIN", "TL_ASSET."
FORMAT_VERSION = 1
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<?", U64: "<Q", I64: "<q", F64: "<d"}
_NP = {U8: np.uint8, I8: np.int8, U16: np.uint16, I16: np.int16, U32: np.uint32, I32: np.int32, F32: np.float32,
       BOOL: np.bool_, U64: np.uint64, I64: np.int64, F64: np.float64}


@dataclass
class TensorInfo:
    name: str
    ty: int                 # ggml type
    ne: list[int]           # ggml order: ne[0] is the row length
    offset: int             # into the data section
    nbytes: int


class GgufError(ValueError):
    pass


class GgufFile:
    """Read side. `tensor_bytes(i)` is a zero-copy view into the mapped file."""

    def __init__(self, path: str) -> None:
        self.path = path
        self._f = open(path, "rb")
        self._m = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._p = 0
        magic, self.version = self._unpack("<II")
        if magic != MAGIC:
            raise GgufError("%s is not a GGUF file" % path)
        if self.version not in (2, 3):
            raise GgufError("GGUF version %d is not supported" % self.version)
        n_tensors, n_kv = self._unpack("<QQ")
        self.kv: dict[str, tuple[int, object]] = {}
        for _ in range(n_kv):
            key = self._string()
            (ty,) = self._unpack("<I")
            self.kv[key] = (ty, self._value(ty))
        self.tensors: list[TensorInfo] = []
        for _ in range(n_tensors):
            name = self._string()
            (rank,) = self._unpack("<I")
            ne = list(self._unpack("<%dQ" % rank)) if rank else []
            ty, off = self._unpack("<IQ")
            rows = int(np.prod(ne[1:], dtype=np.int64)) if len(ne) > 1 else 1
            nbytes = row_size(ty, ne[0]) * rows if ne else 0
            self.tensors.append(TensorInfo(name, ty, ne, off, nbytes))
        self.alignment = int(self.kv.get("general.alignment", (U32, 32))[1])
        self.data_offset = (self._p + self.alignment - 1) // self.alignment * self.alignment

    def close(self) -> None:
        try:
            self._m.close()
        except BufferError:
            pass   # tensor views handed out by tensor_bytes() still exist: the mapping goes away with the last of them
        self._f.close()

    def _unpack(self, fmt: str):
        n = struct.calcsize(fmt)
        if self._p + n > len(self._m):
            raise GgufError("truncated GGUF file")
        v = struct.unpack_from(fmt, self._m, self._p)
        self._p += n
        return v

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        if self._p + n > len(self._m):
            raise GgufError("truncated GGUF file")
        s = self._m[self._p:self._p + n].decode("utf-8")
        self._p += n
        return s

    def _value(self, ty: int):
        if ty == STRING:
            return self._string()
        if ty == ARRAY:
            et, n = self._unpack("<IQ")
            if et == STRING:
                return [self._string() for _ in range(n)]
            if et not in _NP:
                raise GgufError("array of type %d" % et)
            a = np.frombuffer(self._m, _NP[et], n, self._p).copy()
            self._p += a.nbytes
            return a
        if ty not in _SCALAR:
            raise GgufError("value of type %d" % ty)
        return self._unpack(_SCALAR[ty])[0]

    # ---- tensorlisp conventions
    def program(self) -> str:
        """The Scheme program of the file (gguf.rs:136-153)."""
        ver = self.kv.get(TL_VER)
        if ver is None:
            raise GgufError("not a tensorlisp file: %s is missing" % TL_VER)
        if ver[1] != FORMAT_VERSION:
            raise GgufError("%s is %d, this runtime supports version %d" % (TL_VER, ver[1], FORMAT_VERSION))
        if TL_TXT in self.kv:
            return self.kv[TL_TXT][1]
        if TL_BIN in self.kv:
            raise GgufError("binary programs (%s) are not supported yet" % TL_BIN)
        raise GgufError("no program: neither %s nor %s is set" % (TL_TXT, TL_BIN))

    def assets(self) -> dict[str, bytes]:
        return {k[len(TL_ASSET_PREFIX):]: bytes(v[1]) for k, v in self.kv.items()
                if k.startswith(TL_ASSET_PREFIX) and v[0] == ARRAY}

    def tensor_bytes(self, i: int) -> np.ndarray:
        t = self.tensors[i]
        return np.frombuffer(self._m, np.uint8, t.nbytes, self.data_offset + t.offset)

    def tensor_file_offset(self, i: int) -> int:
        return self.data_offset + self.tensors[i].offset


class GgufWriter:
    def __init__(self, alignment: int = 32) -> None:
        self.alignment = alignment
        self.kv: list[tuple[str, int, object]] = []
        self.tensors: list[tuple[str, int, list[int], np.ndarray]] = []

    def _set(self, key: str, ty: int, value) -> None:
        self.kv = [e for e in self.kv if e[0] != key] + [(key, ty, value)]

    def set_str(self, key: str, value: str) -> None:
        self._set(key, STRING, value)

    def set_u32(self, key: str, value: int) -> None:
        self._set(key, U32, int(value))

    def set_bytes(self, key: str, data: bytes) -> None:
        self._set(key, ARRAY, np.frombuffer(bytes(data), np.uint8))

    def set_program(self, text: str) -> None:   # gguf.rs:396-403
        self.kv = [e for e in self.kv if e[0] != TL_BIN]
        self.set_u32(TL_VER, FORMAT_VERSION)
        self.set_str(TL_TXT, text)

    def set_asset(self, name: str, data: bytes) -> None:
        self.set_bytes(TL_ASSET_PREFIX + name, data)

    def copy_metadata(self, src: GgufFile) -> None:
        for k, (ty, v) in src.kv.items():
            self._set(k, ty, v)

    def add_tensor(self, name: str, ty: int, ne: list[int], data: np.ndarray) -> None:
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        rows = int(np.prod(ne[1:], dtype=np.int64)) if len(ne) > 1 else 1
        if data.nbytes != row_size(ty, ne[0]) * rows:
            raise GgufError("tensor %s: %d bytes for type %d shape %s" % (name, data.nbytes, ty, ne))
        self.tensors.append((name, ty, list(ne), data))

    @staticmethod
    def _str(s: str) -> bytes:
        b = s.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def _val(self, ty: int, v) -> bytes:
        if ty == STRING:
            return self._str(v)
        if ty == ARRAY:
            if isinstance(v, list):
                return struct.pack("<IQ", STRING, len(v)) + b"".join(self._str(s) for s in v)
            v = np.ascontiguousarray(v)
            et = {np.dtype(d): t for t, d in _NP.items()}[v.dtype]
            return struct.pack("<IQ", et, v.size) + v.tobytes()
        return struct.pack(_SCALAR[ty], v)

    def write(self, path: str) -> None:
        al = self.alignment
        head = struct.pack("<IIQQ", MAGIC, 3, len(self.tensors), len(self.kv))
        for k, ty, v in self.kv:
            head += self._str(k) + struct.pack("<I", ty) + self._val(ty, v)
        off = 0
        offsets = []
        for name, ty, ne, data in self.tensors:
            offsets.append(off)
            head += self._str(name) + struct.pack("<I", len(ne)) + struct.pack("<%dQ" % len(ne), *ne) + struct.pack("<IQ", ty, off)
            off += (data.nbytes + al - 1) // al * al
        with open(path, "wb") as f:
            f.write(head)
            f.write(b"\0" * ((len(head) + al - 1) // al * al - len(head)))
            for (_, _, _, data), o in zip(self.tensors, offsets):
                f.write(data.tobytes())
                f.write(b"\0" * ((data.nbytes + al - 1) // al * al - data.nbytes))


# ------------------------------------------------------------------ `tl quantize`
VIEW_OPS = ("RESHAPE", "VIEW", "PERMUTE", "TRANSPOSE")   # uses of their result count as uses of their source
QUANTIZABLE_USES = (("MUL_MAT", 0), ("MUL_MAT_ID", 0), ("GET_ROWS", 0), ("IM2COL", 0))   # (op, source index) that take quantized weights


def glob_match(pattern: str, name: str) -> bool:
    """`*` and `?` globs over the whole name (crates/tensorlisp-cli/src/common.rs:236-257)."""
    import re
    rx = "".join(".*" if c == "*" else "." if c == "?" else re.escape(c) for c in pattern)
    return re.fullmatch(rx, name, flags=re.S) is not None


def weight_uses(graphs) -> dict:
    """Every (op, source index) that consumes each weight tensor (by name) in any of the graphs, looking through
    view ops (crates/tensorlisp-cli/src/quantize.rs:59-80): a weight is used however any entry uses it."""
    from . import graph as G

    uses: dict[str, list] = {}
    for g in graphs:
        def weight_of(t: int):
            T = g.tensors[t]
            seen = 0
            # the builder resolves views to their root (`view_src`); a chain of view NODES is followed through src[0]
            while True:
                root = g.tensors[T.view_src] if T.view_src >= 0 else T
                if root.storage_kind == G.WEIGHT and root.op == "NONE":
                    return root.name
                if T.op in VIEW_OPS and T.src[0] >= 0 and seen < 64:
                    T = g.tensors[T.src[0]]
                    seen += 1
                    continue
                return None
        for t in g.nodes:
            T = g.tensors[t]
            is_view = T.op in VIEW_OPS
            for j, s in enumerate(T.src):
                if s < 0:
                    continue
                w = weight_of(s)
                if w is not None and not (is_view and j == 0):
                    uses.setdefault(w, []).append((T.op, j))
    return uses


def skip_reason(t, target: int, uses, include=(), exclude=(), min_elements: int = 1024, include_1d: bool = False,
                requantize: bool = False):
    """Why a tensor keeps its type, or None to convert it: the rules and the wording of
    crates/tensorlisp-cli/src/quantize.rs:148-191, in the same order."""
    from . import graph as G

    tname = lambda ty: G.TYPE_TRAITS[ty][0]
    elements = int(np.prod(t.ne, dtype=np.int64)) if t.ne else 1
    if t.ty == target:
        return "already %s" % tname(target)
    if include and not any(glob_match(g, t.name) for g in include):
        return "not included"
    for g in exclude:
        if glob_match(g, t.name):
            return "excluded by %s" % g
    if tname(t.ty) in ("i8", "i16", "i32", "i64"):
        return "integer tensor"
    if uses is not None:
        lst = uses.get(t.name)
        if lst is None:
            return "not used by the program"
        for op, j in lst:
            if (op, j) not in QUANTIZABLE_USES:
                return "used by %s (source %d); only matmul/get-rows weights are quantized" % (op, j)
    if G.TYPE_TRAITS[t.ty][1] > 1 and not requantize:
        return "already quantized (use --requantize)"
    if len(t.ne) < 2 and not include_1d:
        return "1-D (use --include-1d)"
    if elements < min_elements:
        return "fewer than %d elements" % min_elements
    row = t.ne[0] if t.ne else 1
    blck = G.TYPE_TRAITS[target][1]
    if row % blck != 0:
        return "row length %d is not a multiple of the %s block size %d" % (row, tname(target), blck)
    return None


def _to_f32(native, t, raw: np.ndarray) -> np.ndarray:
    """The tensor's values as f32 rows (DType::to_f32): plain types on the host, block-quantized ones through a
    one-node program (CPY with a dequantizing read) on the GPU."""
    from . import graph as G
    from .native import Native, NativeProgram

    rows = int(np.prod(t.ne[1:], dtype=np.int64)) if len(t.ne) > 1 else 1
    if t.ty == G.F32:
        return raw.view(np.float32).reshape(rows, t.ne[0])
    if t.ty == G.F16:
        return raw.view(np.float16).astype(np.float32).reshape(rows, t.ne[0])
    if t.ty == G.BF16:
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(rows, t.ne[0])
    g = G.Graph()
    w = g.weight(t.ty, [t.ne[0], rows], t.name)
    y = g.output(g.cast(w, G.F32, "values"))
    n = Native.load([raw])
    prog = NativeProgram.compile(n, g)
    prog.run()
    out = prog.read(y).reshape(rows, t.ne[0]).copy()
    prog.free()
    n.close()
    return out


def quantize_file(native, src_path: str, dst_path: str, ty: int, graphs=None, include=(), exclude=(), min_elements: int = 1024,
                  include_1d: bool = False, requantize: bool = False) -> list[dict]:
    """`tl quantize` (crates/tensorlisp-cli/src/quantize.rs:193-267) with the rows quantized ON THE GPU. With `graphs`
    (the program's entries as Graph objects; the reference builds them from the Scheme program stored in the file)
    only weights whose every use is source 0 of MUL_MAT / MUL_MAT_ID / GET_ROWS / IM2COL are converted, seen through
    view ops; without, tensors are chosen by name, rank and size only (`--no-graph`). Everything else and all metadata
    are copied. Returns the report: one dict per tensor (name, from, to, shape, bytes_before, bytes_after, kept_because)."""
    from . import graph as G
    from .native import quantize_rows

    if src_path == dst_path:
        raise GgufError("output must differ from input")
    src = GgufFile(src_path)
    out = GgufWriter(src.alignment)
    out.copy_metadata(src)
    uses = weight_uses(graphs) if graphs is not None else None
    report = []
    for i, t in enumerate(src.tensors):
        raw = src.tensor_bytes(i)
        reason = skip_reason(t, ty, uses, include, exclude, min_elements, include_1d, requantize)
        if reason is None:
            data = quantize_rows(native, ty, np.ascontiguousarray(_to_f32(native, t, raw)))
            out.add_tensor(t.name, ty, t.ne, data)
            after = int(data.nbytes)
        else:
            out.add_tensor(t.name, t.ty, t.ne, raw)
            after = int(t.nbytes)
        report.append({"name": t.name, "from": G.TYPE_TRAITS[t.ty][0], "to": G.TYPE_TRAITS[ty if reason is None else t.ty][0],
                       "shape": list(t.ne), "bytes_before": int(t.nbytes), "bytes_after": after, "kept_because": reason})
    out.write(dst_path)
    src.close()
    return report


# ------------------------------------------------------------------ `tl convert`
# safetensors dtype -> (numpy dtype, bytes per element)
_ST_TYPES = {"F64": (np.float64, 8), "F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2), "I64": (np.int64, 8),
             "I32": (np.int32, 4), "I16": (np.int16, 2), "I8": (np.int8, 1), "U32": (np.uint32, 4), "U16": (np.uint16, 2), "U8": (np.uint8, 1),
             "BOOL": (np.uint8, 1)}
_ST_FLOAT = ("F64", "F32", "F16", "BF16")


def read_safetensors_header(path: str):
    """(entries, data start): every tensor of a .safetensors file as {name, dtype, shape, start, end} in file order of
    their data, offsets relative to the data section (the format: u64 header length, JSON header, data)."""
    import json
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
    entries = [{"name": k, "dtype": v["dtype"], "shape": [int(d) for d in v["shape"]], "start": int(v["data_offsets"][0]),
                "end": int(v["data_offsets"][1])} for k, v in header.items() if k != "__metadata__"]
    entries.sort(key=lambda e: e["start"])
    return entries, 8 + n


def parse_type(name: str) -> int:
    from . import graph as G
    for ty, (n, _, _) in G.TYPE_TRAITS.items():
        if n.lower() == name.lower():
            return ty
    raise GgufError("unknown type %r" % name)


def convert_target(dtype: str):
    """--dtype of `tl convert` (crates/tensorlisp-cli/src/convert.rs:227-237): ("keep", None), ("float", type) or
    ("quant", type)."""
    from . import graph as G
    if dtype == "keep":
        return ("keep", None)
    if dtype in ("f32", "f16", "bf16"):
        return ("float", parse_type(dtype))
    try:
        ty = parse_type(dtype)
    except GgufError:
        ty = None
    if ty is None or G.TYPE_TRAITS[ty][1] == 1:
        raise GgufError("unknown --dtype %r (expected keep, f32, f16, bf16 or a quantized type such as q8_0, q4_0, q4_K)" % dtype)
    return ("quant", ty)


def stored_type(st_dtype: str, ndim: int, target, quant_ok: bool):
    """The type a safetensors tensor is stored as (convert.rs:129-149): with anything but f32, 1-D float tensors stay f32;
    a quantized target applies where `quant_ok`, other matrices become f16; integers become i8 / i16 / i32."""
    from . import graph as G
    kind, ty = target

    def float_type(native: int) -> int:
        if kind == "keep":
            return native
        if kind == "float":
            return G.F32 if ndim <= 1 and ty != G.F32 else ty
        if ndim <= 1:
            return G.F32
        return ty if quant_ok else G.F16

    if st_dtype in ("F32", "F64"):
        return float_type(G.F32)
    if st_dtype == "F16":
        return float_type(G.F16)
    if st_dtype == "BF16":
        return float_type(G.BF16)
    if st_dtype == "I8":
        return G.I8
    if st_dtype == "I16":
        return G.I16
    if st_dtype in ("I32", "I64", "U32", "U16", "U8", "BOOL"):
        return G.I32
    return None


def _split_assignment(s: str):
    if "=" not in s:
        raise GgufError("expected NAME=VALUE, got %r" % s)
    k, v = s.split("=", 1)
    return k, v


def convert_name(name: str, strip_prefix=(), replace_prefix=(), rename=()) -> str:
    """convert.rs:217-224: the first matching prefix is stripped, then the first matching prefix replaced, then an exact
    rename applied."""
    stripped = next((name[len(p):] for p in strip_prefix if name.startswith(p)), name)
    replaced = next((new + stripped[len(old):] for old, new in replace_prefix if stripped.startswith(old)), stripped)
    return next((new for old, new in rename if old == replaced), replaced)


def convert_plan(entries, dtype: str = "keep", types=(), no_quant=(), min_elements: int = 1024, include=(), exclude=(),
                 strip_prefix=(), replace_prefix=(), rename=(), offset=()):
    """What `tl convert` does with every tensor, decided before any data is read (convert.rs:271-302): a list of
    {name, new_name, dtype, shape, stored, offset} for the converted tensors and the list of skipped names."""
    from . import graph as G
    target = convert_target(dtype)
    type_rules = [(g, parse_type(t)) for g, t in map(_split_assignment, types)]
    offsets = [(g, float(v)) for g, v in map(_split_assignment, offset)]
    renames = [_split_assignment(r) for r in rename]
    prefixes = [_split_assignment(r) for r in replace_prefix]
    plan, skipped = [], []
    for e in entries:
        name, st, shape = e["name"], e["dtype"], e["shape"]
        if (include and not any(glob_match(g, name) for g in include)) or any(glob_match(g, name) for g in exclude):
            skipped.append(name)
            continue
        is_float = st in _ST_FLOAT
        elements = int(np.prod(shape, dtype=np.int64)) if shape else 1
        quant_ok = False
        if target[0] == "quant":
            blck = G.TYPE_TRAITS[target[1]][1]
            quant_ok = (is_float and elements >= min_elements and bool(shape) and shape[-1] % blck == 0
                        and not any(glob_match(g, name) for g in no_quant))
        stored = stored_type(st, len(shape), target, quant_ok)
        if stored is None:
            raise GgufError("tensor %s: unsupported safetensors dtype %s" % (name, st))
        if is_float:
            stored = next((ty for g, ty in type_rules if glob_match(g, name)), stored)
        row = shape[-1] if shape else 1
        if row % G.TYPE_TRAITS[stored][1] != 0:
            raise GgufError("tensor %s: rows of %d values do not fit the blocks of %s" % (name, row, G.TYPE_TRAITS[stored][0]))
        if st in _ST_TYPES and e["end"] - e["start"] != elements * _ST_TYPES[st][1]:
            raise GgufError("tensor %s: %d bytes of data do not match shape %s" % (name, e["end"] - e["start"], shape))
        off = next((v for g, v in offsets if glob_match(g, name)), None)
        if off is not None and not is_float:
            raise GgufError("--offset matches %s, which is not a float tensor" % name)
        plan.append({"name": name, "new_name": convert_name(name, strip_prefix, prefixes, renames), "dtype": st, "shape": list(shape),
                     "stored": stored, "offset": off, "start": e["start"], "end": e["end"]})
    return plan, skipped


def convert_safetensors(native, inputs, dst_path: str, dtype: str = "keep", program: str | None = None, assets=(), meta=(), **rules):
    """`tl convert` (crates/tensorlisp-cli/src/convert.rs:226-330) for local .safetensors files, with float tensors encoded
    ON THE GPU (`tlb_quantize_rows`: f16, bf16 and every block type it takes; bit-exact with the reference's
    DType::from_f32). `rules` are convert_plan's keyword arguments. Tensors keep the order of the files. Returns the report:
    one dict per tensor (name, new_name, from, to, shape, bytes) plus the skipped names."""
    from . import graph as G
    from .native import quantize_rows

    out = GgufWriter()
    if program is not None:
        out.set_program(program)
    for m in meta:
        k, v = _split_assignment(m)
        out.set_str(k, v)
    for name, data in assets:
        out.set_asset(name, data)
    report, all_skipped = [], []
    for path in ([inputs] if isinstance(inputs, str) else list(inputs)):
        entries, data0 = read_safetensors_header(path)
        plan, skipped = convert_plan(entries, dtype, **rules)
        all_skipped += skipped
        raw = np.memmap(path, np.uint8, "r", offset=data0) if plan else None
        for p in plan:
            st, stored, shape = p["dtype"], p["stored"], p["shape"]
            npdt, _ = _ST_TYPES[st]
            src = np.frombuffer(raw[p["start"]:p["end"]], npdt)
            row = shape[-1] if shape else 1
            native_same = (st, stored) in (("F32", G.F32), ("F16", G.F16), ("BF16", G.BF16), ("I8", G.I8), ("I16", G.I16), ("I32", G.I32))
            if native_same and p["offset"] is None:
                data = src
            elif st in _ST_FLOAT:
                if st == "BF16":
                    vals = (src.astype(np.uint32) << 16).view(np.float32)
                else:
                    vals = src.astype(np.float32)
                if p["offset"] is not None:
                    vals = vals + np.float32(p["offset"])
                data = vals if stored == G.F32 else quantize_rows(native, stored, np.ascontiguousarray(vals.reshape(-1, max(row, 1))))
            else:
                wide = src.astype(np.int64)
                if wide.size and (wide.min() < -2 ** 31 or wide.max() >= 2 ** 31):
                    raise GgufError("tensor %s: a value does not fit in i32" % p["name"])
                data = wide.astype(np.int32)
            ne = list(reversed(shape)) if shape else [1]
            out.add_tensor(p["new_name"], stored, ne, np.ascontiguousarray(data))
            report.append({"name": p["name"], "new_name": p["new_name"], "from": st.lower(), "to": G.TYPE_TRAITS[stored][0], "shape": shape,
                           "bytes": int(np.ascontiguousarray(data).nbytes)})
    out.write(dst_path)
    return {"tensors": report, "skipped": all_skipped}


def pack_program(src_path: str, dst_path: str | None, program: str, assets=()) -> None:
    """`tl pack` (crates/tensorlisp-cli/src/convert.rs:374-397): stores a program (and assets, replacing those of the same
    name) in a GGUF file; every tensor and every other key is carried over. Writes to `dst_path`, or replaces the file.
    The reference first checks that the program is valid by evaluating it; that needs its Scheme front end."""
    import os
    src = GgufFile(src_path)
    out = GgufWriter(src.alignment)
    out.copy_metadata(src)
    out.set_program(program)
    for name, data in assets:
        out.set_asset(name, data)
    for i, t in enumerate(src.tensors):
        out.add_tensor(t.name, t.ty, t.ne, np.array(src.tensor_bytes(i)))
    target = dst_path or src_path
    tmp = target + ".tmp"
    out.write(tmp)
    src.close()
    os.replace(tmp, target)
