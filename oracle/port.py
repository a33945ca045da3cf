"""TEST INFRASTRUCTURE - ctypes access to the plain-C restatement (oracle/quants_port.c, oracle/rans_port.c),
built by `make -C oracle port` into oracle/_build/liboracle.so.  Only tests/, smoke() and bench.py's CPU-baseline
legs may import this; the product never does."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")
PORT_TYPES = {2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 42}     # ggml types the restatement covers
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            subprocess.run(["make", "-C", _HERE, "port"], check=True, capture_output=True)
        L = ctypes.CDLL(_SO)
        L.op_quantize_row.restype = ctypes.c_size_t
        L.op_quantize_row.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        L.op_f32_to_f16.restype = ctypes.c_uint16
        L.op_f32_to_f16.argtypes = [ctypes.c_float]
        L.op_f16_to_f32.restype = ctypes.c_float
        L.op_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.op_nearest_int.restype = ctypes.c_int
        L.op_nearest_int.argtypes = [ctypes.c_float]
        _lib = L
    return _lib


def quantize(ttype, x, imatrix=None):
    """x: float32 (nrows, n_per_row) -> uint8 bytes, row by row"""
    L = lib()
    x = np.ascontiguousarray(x, np.float32)
    nrows, npr = x.shape
    imp = None if imatrix is None else np.ascontiguousarray(imatrix, np.float32)
    probe = np.empty(npr * 2, np.uint8)
    rb = L.op_quantize_row(ttype, x[0].ctypes.data, probe.ctypes.data, npr, None if imp is None else imp.ctypes.data)
    if rb == 0:
        raise ValueError(f"ggml type {ttype} is not covered by the C restatement")
    out = np.empty(nrows * rb, np.uint8)
    for r in range(nrows):
        L.op_quantize_row(ttype, x[r].ctypes.data, out[r * rb:].ctypes.data, npr, None if imp is None else imp.ctypes.data)
    return out
