"""TEST INFRASTRUCTURE - ctypes access to the reference's own C quantisers.

`oracle/_ref/libggmlq_ref.so` is the reference's `seedpack/ggml/ggml-quants.c`, compiled unmodified
by `oracle/Makefile` with a stable sort standing in for qsort (what the reference's authoritative
`--cpu` build does, seedpack/gpuquant.py:70-80, 238-245).  Only tests/, `__graft_entry__.smoke()`
and bench.py's CPU-baseline legs may import this module; the product never does.

Entry points follow seedpack/requant.py:21-27 (`QFUN`) and :114-134 (`quantize`).
"""
import ctypes
import os
import threading
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref", "libggmlq_ref.so")
_REF_V1 = os.path.join(_HERE, "_ref", "libggmlq_ref_v1.so")

# ggml type id -> (name, weights per block, bytes per block)      seedpack/requant.py:21-27
QFUN = {2: ("q4_0", 32, 18), 3: ("q4_1", 32, 20), 6: ("q5_0", 32, 22), 7: ("q5_1", 32, 24),
        8: ("q8_0", 32, 34), 10: ("q2_K", 256, 84), 11: ("q3_K", 256, 110), 12: ("q4_K", 256, 144),
        13: ("q5_K", 256, 176), 14: ("q6_K", 256, 210), 16: ("iq2_xxs", 256, 66), 17: ("iq2_xs", 256, 74),
        18: ("iq3_xxs", 256, 98), 19: ("iq1_s", 256, 50), 20: ("iq4_nl", 32, 18), 21: ("iq3_s", 256, 110),
        22: ("iq2_s", 256, 82), 23: ("iq4_xs", 256, 136), 29: ("iq1_m", 256, 56), 42: ("q2_0", 64, 18),
        # not in the reference's table, but in its ggml-quants.c (lines 40, 350, 384, 2317, 2383)
        34: ("tq1_0", 256, 54), 35: ("tq2_0", 256, 66), 39: ("mxfp4", 32, 17), 40: ("nvfp4", 64, 36), 41: ("q1_0", 128, 18)}
EXTRA = {34, 35, 39, 40, 41}
IQ2_INIT = {16, 17, 19, 22, 29}            # need iq2xs_init_impl(type)   seedpack/requant.py:28
IQ3_INIT = {18: 256, 21: 512}              # need iq3xs_init_impl(grid)   seedpack/requant.py:29
NEEDS_IMATRIX = {16, 17, 19}       # assert quant_weights (ggml-quants.c:3303, 3481, 4521 ...)

_libs = {}
_lock = threading.Lock()
_inited = set()


def available():
    return os.path.exists(_REF)


def _lib(variant=0):
    path = _REF if variant == 0 else _REF_V1
    with _lock:
        if path not in _libs:
            if not os.path.exists(path):
                raise RuntimeError(f"{path} is missing: run `make -C oracle ref` where the reference tree is mounted")
            L = ctypes.CDLL(path)
            for name, _, _ in QFUN.values():
                f = getattr(L, "quantize_" + name)
                f.restype = ctypes.c_size_t
                f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
                g = getattr(L, "dequantize_row_" + name)
                g.restype = None
                g.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
            L.iq2xs_init_impl.argtypes = [ctypes.c_int]
            L.iq3xs_init_impl.argtypes = [ctypes.c_int]
            _libs[path] = L
        return _libs[path]


def _init(t, variant):
    L = _lib(variant)
    with _lock:
        if (t, variant) in _inited:
            return
        if t in IQ2_INIT:
            L.iq2xs_init_impl(t)
        if t in IQ3_INIT:
            L.iq3xs_init_impl(IQ3_INIT[t])
        _inited.add((t, variant))


def bf16_to_f32(bits):
    """uint16 bf16 bit patterns -> float32 (exact)"""
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize(ttype, x, imatrix=None, variant=0, threads=None):
    """x: float32 (nrows, n_per_row) -> uint8 bytes of the whole tensor, row by row exactly as the
    reference's per-row launch does (seedpack/gpuquant.py:206-211: quantize_<t>(row, dst, 1, npr, w))."""
    name, qk, bs = QFUN[ttype]
    _init(ttype, variant)
    L = _lib(variant)
    x = np.ascontiguousarray(x, np.float32)
    nrows, npr = x.shape
    assert npr % qk == 0
    rb = npr // qk * bs
    out = np.empty(nrows * rb, np.uint8)
    imp = None if imatrix is None else np.ascontiguousarray(imatrix, np.float32)
    if imp is not None:
        assert imp.size == npr
    f = getattr(L, "quantize_" + name)
    threads = threads or os.cpu_count() or 1
    chunk = max(1, (nrows + threads * 4 - 1) // (threads * 4))

    def run(r0):
        r1 = min(nrows, r0 + chunk)
        for r in range(r0, r1):          # one row per call, like the reference's kernel
            f(x[r].ctypes.data, out[r * rb:(r + 1) * rb].ctypes.data, 1, npr,
              None if imp is None else imp.ctypes.data)

    if threads == 1 or nrows == 1:
        run(0) if chunk >= nrows else [run(r0) for r0 in range(0, nrows, chunk)]
    else:
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(run, range(0, nrows, chunk)))
    return out


def dequantize(ttype, y, n_weights):
    """quantised bytes -> float32 with the reference's dequantize_row_<type>"""
    name, qk, bs = QFUN[ttype]
    L = _lib(0)
    y = np.ascontiguousarray(y, np.uint8)
    out = np.empty(n_weights, np.float32)
    getattr(L, "dequantize_row_" + name)(y.ctypes.data, out.ctypes.data, n_weights)
    return out


def iq_table(kind, index, which, count):
    """raw view of the grids / maps / neighbour lists the reference's init functions built
    (seedpack/ggml/export.c:6-11); kind = 2 or 3, which = 0 grid, 1 map, 2 neighbours"""
    L = _lib(0)
    fn = L.vq_iq2_table if kind == 2 else L.vq_iq3_table
    fn.restype = ctypes.c_void_p
    fn.argtypes = [ctypes.c_int, ctypes.c_int]
    ptr = fn(index, which)
    ctype = {0: ctypes.c_uint64 if kind == 2 else ctypes.c_uint32, 1: ctypes.c_int32, 2: ctypes.c_uint16}[which]
    return np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctype)), (count,)).copy()
