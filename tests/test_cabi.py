"""The C-ABI library loads and exports every symbol the header declares.
No compute call is made here (no GPU needed)."""
import ctypes
import os
import re

from conftest import ROOT
from rwkv_quant_b200 import _lib


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            src = open(os.path.join(inc, f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names |= set(re.findall(r"\b(rwkvq_[a-z0-9_]+)\s*\(", src))
    return names


def test_library_exports_header_symbols():
    lib = _lib.load()
    declared = _declared()
    assert declared, "no declarations found in include/*.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(_lib.exported_symbols()), \
        "ctypes prototypes and the header disagree: " + str(declared ^ set(_lib.exported_symbols()))


def test_error_strings_and_struct_layout():
    lib = _lib.load()
    assert lib.rwkvq_abi_version() >= 1
    assert lib.rwkvq_strerror(0) == b"ok"
    assert b"shape" in lib.rwkvq_strerror(-1)
    # rwkvq_qtensor: six int32 then eleven pointers
    assert ctypes.sizeof(_lib.QTensorStruct) == 6 * 4 + 11 * 8
    assert _lib.QTensorStruct.codes.offset == 24


def test_argument_validation_without_gpu():
    """Null / malformed descriptors are refused before any CUDA call."""
    lib = _lib.load()
    assert lib.rwkvq_dequant(None, None, 0, 0, None) == -7
    t = _lib.QTensorStruct(kind=1, bits=4, rows=8, cols=100, gs=32, sb=8)
    t.codes = 0x1000
    assert lib.rwkvq_dequant(ctypes.byref(t), 0x1000, 0, 0, None) == -1      # IN % 256
    assert b"256" in lib.rwkvq_last_error_detail()
    t = _lib.QTensorStruct(kind=9, bits=4, rows=8, cols=256, gs=32, sb=8)
    t.codes = 0x1000
    assert lib.rwkvq_gemv(ctypes.byref(t), 0x1000, 0, 1, 256, 0x1000, 8, 0, None, None) == -3
