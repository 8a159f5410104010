"""The C-ABI library loads and exports every symbol include/llmp_b200.h
declares; without a B200 its launch entry points refuse instead of falling
back."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "llmp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llmp_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from llmp_b200 import _native
    lib = C.CDLL(_native.LIB_PATH)
    names = _declared()
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_native.SIGNATURES) == names


def test_no_fallback_without_a_device():
    import torch
    from llmp_b200 import _native
    L = _native.lib()
    if torch.cuda.is_available():
        return
    assert L.llmp_b200_available() == 0
    assert L.llmp_b200_sm_count() == 0
    d = _native.VecQDesc()
    assert L.llmp_b200_vecq(_native.TYPE_Q4_K, C.byref(d), -1, None) == _native.REJECTED
    assert b"vecq" in L.llmp_b200_last_error()
    assert L.llmp_b200_q8_1_row_blocks(2560) == 80
    assert L.llmp_b200_vecq_variants() >= 1
