"""Residual of a stored quantised tensor against its prediction, on the device - host-side mirror of the
reference's NumPy helpers (seedpack/repo3.py:456-510) over the seedgrow C ABI.

    xor_(r, p)            r ^= p in place, returns the number of non-zero bytes left   (_xor_async + _nonzero)
    count_diff(a, b)      bytes where a and b differ; b None: non-zero bytes of a      (_count_diff)
    xor3(a, b, c)         (a ^ b ^ c as a new tensor, its non-zero byte count)         (_xor3)
    block_ne(f, p, bs)    per-block "differs" flags and their count                     (qr.same)

Counts come back as Python ints (one synchronisation each); pass sync=False to get the device counter
tensor instead and read several of them after one synchronisation.
"""
import ctypes

import torch

from . import _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _u8(t):
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("residual operands must be contiguous CUDA tensors")
    return t.view(torch.uint8).reshape(-1)


def _xor(a, b, c, out, sync):
    a = _u8(a)
    n = a.numel()
    for t in (b, c, out):
        if t is not None and _u8(t).numel() != n:
            raise ValueError("operands differ in size")
    cnt = torch.zeros(1, dtype=torch.int64, device=a.device)
    rc = _lib.lib().sg_residual_xor(a.device.index, _stream(a.device), _p(a), _p(None if b is None else _u8(b)),
                                    _p(None if c is None else _u8(c)), _p(None if out is None else _u8(out)), n, _p(cnt))
    _lib.check(rc, "sg_residual_xor")
    return int(cnt.item()) if sync else cnt


def xor_(r, p, sync=True):
    return _xor(r, p, None, r, sync)


def count_diff(a, b=None, sync=True):
    return _xor(a, b, None, None, sync)


def xor3(a, b, c, sync=True):
    out = torch.empty_like(_u8(a))
    return out, _xor(a, b, c, out, sync)


def block_ne(file, pred, block_bytes, sync=True, flags=True):
    f, p = _u8(file), _u8(pred)
    if f.numel() != p.numel() or f.numel() % block_bytes:
        raise ValueError("sizes must match and be whole blocks")
    nb = f.numel() // block_bytes
    ne = torch.empty(nb, dtype=torch.uint8, device=f.device) if flags else None
    cnt = torch.zeros(1, dtype=torch.int64, device=f.device)
    rc = _lib.lib().sg_residual_blocks(f.device.index, _stream(f.device), _p(f), _p(p), block_bytes, nb, _p(ne), _p(cnt))
    _lib.check(rc, "sg_residual_blocks")
    return ne, (int(cnt.item()) if sync else cnt)
