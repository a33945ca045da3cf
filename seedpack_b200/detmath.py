"""Deterministic float64 helpers on the device - host-side mirror of seedpack/detmath.py (log2, exp2, rows, cols,
total; :178-215) over the seedgrow C ABI.  Same names and argument meanings; arrays are torch CUDA tensors."""
import ctypes

import torch

from . import _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _st(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _f64(x):
    return x.to(torch.float64).contiguous()


def log2(x):
    x = _f64(x)
    y = torch.empty_like(x)
    _lib.check(_lib.lib().sg_dm_log2(x.device.index, _st(x.device), _p(x), x.numel(), _p(y)), "sg_dm_log2")
    return y


def exp2(x):
    x = _f64(x)
    y = torch.empty_like(x)
    _lib.check(_lib.lib().sg_dm_exp2(x.device.index, _st(x.device), _p(x), x.numel(), _p(y)), "sg_dm_exp2")
    return y


def rows(x, square=False):
    x = x.to(torch.float32).contiguous()
    nr, nc = x.shape
    out = torch.empty(nr, dtype=torch.float64, device=x.device)
    _lib.check(_lib.lib().sg_dm_rows(x.device.index, _st(x.device), _p(x), nr, nc, int(square), _p(out)), "sg_dm_rows")
    return out


def cols(x, square=False, mask=None):
    x = x.to(torch.float32).contiguous()
    nr, nc = x.shape
    m = None if mask is None else mask.to(torch.uint8).contiguous()
    out = torch.empty(nc, dtype=torch.float64, device=x.device)
    _lib.check(_lib.lib().sg_dm_cols(x.device.index, _st(x.device), _p(x), nr, nc, int(square), _p(m), _p(out)), "sg_dm_cols")
    return out


def total(x, square=False):
    return rows(x.reshape(1, -1), square)[0]
