"""The C-ABI library loads without a GPU, exports every symbol include/tlb200.h declares, and
fails loudly (never falls back) when no device is present. No compute calls here."""
import ctypes as C
import os
import re

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
