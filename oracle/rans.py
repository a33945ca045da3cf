"""TEST INFRASTRUCTURE - Python access to oracle/rans_port.c (the CPU restatement of the reference's rANS coder)."""
import ctypes

import numpy as np

from . import port


def _lib():
    L = port.lib()
    if not hasattr(L, "_rans_ready"):
        L.op_rans_encode.restype = ctypes.c_size_t
        L.op_rans_encode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        L.op_rans_decode.restype = ctypes.c_int
        L.op_rans_decode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L._rans_ready = True
    return L


def encode(sym, block_tab, block_len, seg_len, freq_full, pb=12):
    """-> (stream uint8, offsets uint64 [nseg + 1])"""
    sym = np.ascontiguousarray(sym, np.uint8)
    bt = np.ascontiguousarray(block_tab, np.uint16)
    f = np.ascontiguousarray(freq_full, np.uint16)
    nseg = (len(sym) + seg_len - 1) // seg_len
    out = np.empty(len(sym) * 2 + 64 * nseg + 64, np.uint8)
    tmp = np.empty(seg_len * 2 + 64, np.uint8)
    off = np.zeros(nseg + 1, np.uint64)
    n = _lib().op_rans_encode(sym.ctypes.data, bt.ctypes.data, block_len, len(sym), seg_len, pb, f.ctypes.data, out.ctypes.data,
                              out.size, off.ctypes.data, tmp.ctypes.data, tmp.size)
    assert n != ctypes.c_size_t(-1).value
    return out[:n].copy(), off


def decode(stream, off, block_tab, block_len, nsym, seg_len, freq_full, pb=12):
    stream = np.ascontiguousarray(stream, np.uint8)
    off = np.ascontiguousarray(off, np.uint64)
    bt = np.ascontiguousarray(block_tab, np.uint16)
    f = np.ascontiguousarray(freq_full, np.uint16)
    out = np.empty(nsym, np.uint8)
    rc = _lib().op_rans_decode(stream.ctypes.data, off.ctypes.data, bt.ctypes.data, block_len, nsym, seg_len, pb, f.ctypes.data, out.ctypes.data)
    return out, rc
