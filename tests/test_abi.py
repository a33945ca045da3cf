"""The C-ABI library loads and exports every symbol include/seedgrow.h declares (no GPU needed)."""
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_header_symbols_are_exported_and_bound():
    from seedpack_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "seedgrow.h")).read()
    declared = set(re.findall(r"SG_API[^;(]*?\b(sg_\w+)\s*\(", hdr))
    assert declared, "no declarations found"
    L = _lib.lib()
    for name in declared:
        assert hasattr(L, name), f"{name} is declared but not exported"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))


def test_type_table():
    import ctypes
    from seedpack_b200 import _lib
    from seedpack_b200.requant import QFUN
    L = _lib.lib()
    for t, (_, qk, bs) in QFUN.items():
        a, b = ctypes.c_int(), ctypes.c_int()
        assert L.sg_type_info(t, ctypes.byref(a), ctypes.byref(b)) == 0
        assert (a.value, b.value) == (qk, bs)
    assert L.sg_type_info(9, None, None) == 2
    assert L.sg_status_string(0) == b"ok"


def test_argument_errors_need_no_gpu():
    """validation happens before any CUDA call"""
    import ctypes
    from seedpack_b200 import _lib
    L = _lib.lib()
    t = (_lib.sg_tensor * 1)()
    t[0].x_off, t[0].y_off, t[0].w_off, t[0].n_rows, t[0].n_per_row = 0, 0, -1, 1, 100
    assert L.sg_quantize_tensors(0, None, 999, 0, ctypes.c_void_p(16), 0, ctypes.c_void_p(16), None, t, 1, None, 0) == 2     # type
    assert L.sg_quantize_tensors(0, None, 8, 1, ctypes.c_void_p(16), 0, ctypes.c_void_p(16), None, t, 1, None, 0) == 2       # variant
    assert L.sg_quantize_tensors(0, None, 8, 0, None, 0, ctypes.c_void_p(16), None, t, 1, None, 0) == 1                       # null x
