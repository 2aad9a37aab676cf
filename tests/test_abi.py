"""The C-ABI library loads without a GPU, exports every symbol include/tlb200.h declares, and
fails loudly (never falls back) when no device is present. No compute calls here."""
import ctypes as C
import os
import re

import numpy as np

import pytest

from tensorlisp_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tlb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tlb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_symbols()
    assert len(names) >= 30
    assert sorted(_lib.SYMBOLS) == names


def test_library_exports_every_symbol():
    L = _lib.lib()
    for name in declared_symbols():
        assert getattr(L, name) is not None


def test_row_size_table():
    L = _lib.lib()
    assert L.tlb_row_size(8, 4096) == 4352     # q8_0: 34 bytes per 32
    assert L.tlb_row_size(2, 4096) == 2304     # q4_0: 18 bytes per 32
    assert L.tlb_row_size(12, 4096) == 2304    # q4_K: 144 bytes per 256
    assert L.tlb_row_size(12, 14336) == 8064
    assert L.tlb_row_size(12, 100) == 0        # not a multiple of the block size
    assert L.tlb_row_size(99, 32) == 0         # unknown type


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = _lib.lib()
    h = C.c_void_p()
    st = L.tlb_device_open(0, C.byref(h))
    assert st == _lib.TLB_NO_DEVICE and not h.value
    assert b"no GPU" in L.tlb_last_error()
    from tensorlisp_b200.native import Native, TlbError
    with pytest.raises(TlbError) as e:
        Native(0)
    assert e.value.kind == "NoDevice"


def test_entry_cache_keeps_eight_shapes_and_drops_the_oldest():
    """Inner::run_native's program cache (crates/tensorlisp/src/model.rs:1049-1068) with a stand-in compiler: one program
    per combination of input shapes, reused on the next call, at most eight per entry, the oldest freed first; entries
    do not share their lists."""
    from tensorlisp_b200.native import EntryCache

    class Prog:
        def __init__(self, log, key):
            self.log, self.key, self.freed = log, key, False

        def free(self):
            self.freed = True
            self.log.append(("free", self.key))

    log = []
    cache = EntryCache(None, build=lambda name, shapes: (name, shapes), compile=lambda native, graph: (log.append(("compile", graph)), Prog(log, graph))[1])
    first = cache.program("decode", ((4096, 1),))
    assert cache.program("decode", ((4096, 1),)) is first and log == [("compile", ("decode", ((4096, 1),)))]
    for n in range(2, 9):
        cache.program("decode", ((4096, n),))
    assert len(cache.programs["decode"]) == 8 and not first.freed
    cache.program("prefill", ((4096, 1),))                       # another entry has its own list
    assert not first.freed
    ninth = cache.program("decode", ((4096, 9),))
    assert first.freed and len(cache.programs["decode"]) == 8 and cache.programs["decode"][-1][1] is ninth
    assert cache.program("decode", ((4096, 1),)) is not first    # dropped: compiled again, and the next oldest goes
    assert ("free", ("decode", ((4096, 2),))) in log
    cache.free()
    assert cache.programs == {} and ninth.freed


def test_i32_inputs_take_whole_numbers_only():
    """model.rs:940-952: an i32 input arrives as f32 values; a fraction, a value out of range or a NaN is an input error
    that names the input."""
    from tensorlisp_b200.native import to_i32
    assert np.array_equal(to_i32("ids", np.array([[0.0, 7.0], [-3.0, 128255.0]], np.float32)), np.array([[0, 7], [-3, 128255]], np.int32))
    assert to_i32("ids", np.array([5, 6], np.int64)).dtype == np.int32
    for bad in (1.5, float("nan"), 3e9, -3e9):
        with pytest.raises(ValueError) as e:
            to_i32("ids", np.array([1.0, bad], np.float32))
        assert "ids" in str(e.value)
