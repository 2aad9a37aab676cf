"""ctypes binding of libtlb200.so (the C ABI declared in include/tlb200.h).

The library is the product: there is no Python or CPU fallback. If it is missing, importing this
module raises with the build command; if there is no GPU, ``tlb_device_open`` fails with
TLB_NO_DEVICE and nothing else can be called.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libtlb200.so"

TLB_OK, TLB_NO_DEVICE, TLB_COMPILE, TLB_PIPELINE, TLB_ALLOC, TLB_EXECUTION, TLB_INVALID, TLB_UNSUPPORTED = range(8)
STATUS_NAMES = ["Ok", "NoDevice", "Compile", "Pipeline", "Alloc", "Execution", "Invalid", "Unsupported"]


class TlbError(RuntimeError):
    """tensorlisp::Error::Backend(String) of the reference (crates/tensorlisp/src/native_ir.rs:11-13)."""

    def __init__(self, status: int, message: str) -> None:
        super().__init__(message)
        self.status = status
        self.kind = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)


class tlb_tensor(C.Structure):
    _fields_ = [
        ("ty", C.c_uint32),
        ("ne", C.c_int64 * 4),
        ("nb", C.c_uint64 * 4),
        ("op", C.c_char * 32),
        ("op_params", C.c_int32 * 16),
        ("src", C.c_int32 * 10),
        ("view_src", C.c_int32),
        ("view_offs", C.c_uint64),
        ("storage_kind", C.c_uint32),
        ("storage_index", C.c_uint32),
        ("name", C.c_char * 64),
    ]


class tlb_graph(C.Structure):
    _fields_ = [
        ("tensors", C.POINTER(tlb_tensor)),
        ("n_tensors", C.c_uint32),
        ("nodes", C.POINTER(C.c_int32)),
        ("n_nodes", C.c_uint32),
        ("keep", C.POINTER(C.c_int32)),
        ("n_keep", C.c_uint32),
    ]


class tlb_leaves(C.Structure):
    _fields_ = [
        ("weight_buffer", C.POINTER(C.c_uint32)),
        ("weight_offset", C.POINTER(C.c_uint64)),
        ("n_weights", C.c_uint32),
        ("state_offset", C.POINTER(C.c_uint64)),
        ("n_states", C.c_uint32),
    ]


# every symbol include/tlb200.h declares: name -> (restype, argtypes)
_P = C.c_void_p
SYMBOLS = {
    "tlb_device_open": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "tlb_device_close": (None, [_P]),
    "tlb_device_name": (C.c_int, [_P, C.c_char_p, C.c_size_t]),
    "tlb_device_sync": (C.c_int, [_P]),
    "tlb_device_stream": (_P, [_P]),
    "tlb_device_sm_count": (C.c_int, [_P]),
    "tlb_last_error": (C.c_char_p, []),
    "tlb_weights_create": (C.c_int, [_P, C.c_uint64, C.POINTER(_P)]),
    "tlb_state_create": (C.c_int, [_P, C.c_uint64, C.POINTER(_P)]),
    "tlb_state_zero": (C.c_int, [_P]),
    "tlb_state_fork": (C.c_int, [_P, C.POINTER(_P)]),
    "tlb_state_copy_blocks": (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, _P, C.c_uint32]),
    "tlb_state_gather_kv": (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, _P, C.c_uint32, _P, C.c_uint32, _P, _P]),
    "tlb_buffer_write": (C.c_int, [_P, C.c_uint64, _P, C.c_uint64]),
    "tlb_buffer_read": (C.c_int, [_P, C.c_uint64, _P, C.c_uint64]),
    "tlb_buffer_size": (C.c_uint64, [_P]),
    "tlb_buffer_device_ptr": (_P, [_P]),
    "tlb_buffer_copy_device": (C.c_int, [_P, C.c_uint64, _P, C.c_uint64]),
    "tlb_buffer_free": (None, [_P]),
    "tlb_program_compile": (C.c_int, [_P, C.POINTER(tlb_graph), C.POINTER(tlb_leaves), C.POINTER(_P), C.c_char_p, C.c_size_t]),
    "tlb_program_free": (None, [_P]),
    "tlb_plan_only": (C.c_int, [C.POINTER(tlb_graph), C.POINTER(tlb_leaves), _P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), _P, _P, _P]),
    "tlb_program_set_input": (C.c_int, [_P, C.c_uint32, _P, C.c_uint64]),
    "tlb_program_feed_input": (C.c_int, [_P, C.c_uint32, C.c_uint32]),
    "tlb_program_run": (C.c_int, [_P, C.POINTER(_P), C.c_uint32, _P]),
    "tlb_program_enqueue": (C.c_int, [_P, C.POINTER(_P), C.c_uint32, _P]),
    "tlb_program_read": (C.c_int, [_P, C.c_uint32, C.c_uint64, _P]),
    "tlb_program_dispatch_count": (C.c_uint32, [_P]),
    "tlb_program_kernel_count": (C.c_uint32, [_P]),
    "tlb_program_label": (C.c_char_p, [_P, C.c_uint32]),
    "tlb_program_tensor_ptr": (_P, [_P, C.c_uint32, C.POINTER(C.c_uint64)]),
    "tlb_program_arena_bytes": (C.c_uint64, [_P]),
    "tlb_program_profile": (C.c_int, [_P, C.POINTER(_P), C.c_uint32, _P, C.POINTER(C.c_float), C.c_uint32]),
    "tlb_quantize_rows": (C.c_int, [_P, C.c_uint32, _P, C.c_int64, C.c_int64, _P]),
    "tlb_quantize_rows_device": (C.c_int, [_P, C.c_uint32, _P, C.c_int64, C.c_int64, _P]),
    "tlb_row_size": (C.c_uint64, [C.c_uint32, C.c_int64]),
    "tlb_paged_attention_static": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_int, C.c_float]),
    "tlb_comm_unique_id": (C.c_int, [_P]),
    "tlb_comm_init": (C.c_int, [_P, C.c_int, C.c_int, _P]),
    "tlb_comm_destroy": (C.c_int, [_P]),
    "tlb_comm_p2p_export": (C.c_int, [_P, _P]),
    "tlb_comm_p2p_import": (C.c_int, [_P, _P]),
    "tlb_program_graph_count": (C.c_uint32, [_P]),
    "tlb_device_comm_generation": (C.c_uint64, [_P]),
    "tlb_comm_p2p_selftest_absent": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_uint32, _P, _P]),
    "tlb_comm_p2p_selftest_rows_absent": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, _P, _P, _P, C.c_float, _P, _P, C.c_uint64]),
    "tlb_selftest_wait_runs_out": (C.c_int, [_P, C.c_uint32, C.c_uint32, C.POINTER(C.c_double)]),
    "tlb_comm_p2p_selftest": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "tlb_comm_p2p_selftest_rows": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, _P, C.c_float, _P, _P, C.c_uint64]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads the shared library; raises loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                "%s is missing: build it with `python -m tensorlisp_b200.build` (needs nvcc, sm_100a). "
                "There is no CPU fallback." % LIB_PATH)
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            f = getattr(L, name)  # AttributeError if the library does not export it
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != TLB_OK:
        raise TlbError(status, lib().tlb_last_error().decode(errors="replace"))
