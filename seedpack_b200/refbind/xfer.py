"""Host <-> device copies of the binding.

The reference moves whole windows of a repository between pageable host memory (files read into NumPy arrays, the
arrays its container writes from) and the device.  A plain copy of pageable memory goes through the driver's own small
staging buffer at a fraction of the link's rate, and a fresh destination array pays a page fault per 4 KiB on one
thread.  Here a large copy is cut into chunks handed to a few worker threads; each has a page-locked slot and a stream
of its own: host memcpy (NumPy releases the GIL) and DMA of different chunks overlap, and a fresh destination is
faulted in by several threads at once.  Page-locked host arrays (the binding's pinned pool) are copied directly.
Both calls return when the data has arrived (CuPy's `set` / `get` semantics)."""
import threading
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

CHUNK = 8 << 20
WORKERS = 6
DIRECT = 4 << 20                   # smaller copies are not worth the hand-over

_pool = None
_pool_lock = threading.Lock()
_local = threading.local()


def _workers():
    global _pool
    if _pool is None:
        with _pool_lock:
            if _pool is None:
                _pool = ThreadPoolExecutor(WORKERS, thread_name_prefix="sg-xfer")
    return _pool


def _slot(device):
    t = _local
    if getattr(t, "device", None) != device:
        torch.cuda.set_device(device)
        t.device, t.stream = device, torch.cuda.Stream(device)
        t.pin = torch.empty(CHUNK, dtype=torch.uint8, pin_memory=True)
        t.np = t.pin.numpy()
    return t


def _up(dst, src, o, n, ready):
    t = _slot(dst.device.index)
    np.copyto(t.np[:n], src[o:o + n])
    with torch.cuda.stream(t.stream):
        t.stream.wait_event(ready)
        dst[o:o + n].copy_(t.pin[:n], non_blocking=True)
    t.stream.synchronize()


def _down(dst, src, o, n, ready):
    t = _slot(src.device.index)
    with torch.cuda.stream(t.stream):
        t.stream.wait_event(ready)
        t.pin[:n].copy_(src[o:o + n], non_blocking=True)
    t.stream.synchronize()
    np.copyto(dst[o:o + n], t.np[:n])


def _pinned(a):
    try:
        return torch.from_numpy(a[:1]).is_pinned() if a.flags.writeable else False
    except Exception:
        return False


def _run(fn, dst, src, n):
    ready = torch.cuda.Event()
    ready.record(torch.cuda.current_stream((dst if fn is _up else src).device))
    fs = [_workers().submit(fn, dst, src, o, min(CHUNK, n - o), ready) for o in range(0, n, CHUNK)]
    for f in fs:
        f.result()


def h2d(dst, src):
    """dst: CUDA uint8 tensor, src: contiguous NumPy uint8 array of the same length; done on return"""
    n = src.size
    if n < DIRECT or _pinned(src):
        if src.flags.writeable:
            dst.copy_(torch.from_numpy(src))
        else:
            import warnings
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                dst.copy_(torch.from_numpy(src))
        return
    _run(_up, dst, src, n)


def d2h(dst, src):
    """dst: contiguous writable NumPy uint8 array, src: CUDA uint8 tensor of the same length; done on return"""
    n = dst.size
    if n < DIRECT or _pinned(dst):
        torch.from_numpy(dst).copy_(src)
        return
    _run(_down, dst, src, n)
