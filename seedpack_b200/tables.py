"""IQ lattice tables: per-device installation and host views (mirror of GPUQuant._upload_tables,
seedpack/gpuquant.py:311-326).  The tables are built inside libseedgrow.so."""
import ctypes

import numpy as np

from . import _lib

NAMES = ("iq2_xxs", "iq2_xs", "iq1", "iq2_s", "iq3_xxs", "iq3_s")


def install(device, stream=None):
    _lib.check(_lib.lib().sg_tables_install(device, ctypes.c_void_p(stream or 0)), "sg_tables_install")


def host(which, what):
    """numpy copy of a built table: what = 0 grid, 1 map, 2 neighbour lists"""
    p, n = ctypes.c_void_p(), ctypes.c_size_t()
    _lib.check(_lib.lib().sg_tables_host(which, what, ctypes.byref(p), ctypes.byref(n)), "sg_tables_host")
    dt = {0: np.uint64 if which < 4 else np.uint32, 1: np.int32, 2: np.uint16}[what]
    buf = (ctypes.c_uint8 * n.value).from_address(p.value)
    return np.frombuffer(buf, dtype=dt).copy()
