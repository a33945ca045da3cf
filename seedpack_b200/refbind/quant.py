"""`GPUQuant` as the reference's repository code calls it (seedpack/gpuquant.py:285-456), served by
seedpack_b200.gpuquant.GPUQuant: same constructor, `quantize_tensors`, `quantize_batch`, `dequantize`, with the
binding's device arrays (refbind.cupy_shim.ndarray) in place of CuPy's.

What differs from the reference's class, by design of the kernels behind it: BF16 / F16 sources are read where they
lie (no float32 staging copy of a launch's tensors, gpuquant.py:396-400), so `max_weights` only bounds how much
output is in flight to the host at a time; there is no source generation, run-time compilation or table file
(gpuquant.py:288-353): the lattice tables are built by the library on first use.
"""
import numpy as np
import torch

from .. import gpuquant as _gq
from ..requant import QFUN
from . import cupy_shim as cp
from . import twins

_TORCH = {np.dtype(np.uint16): torch.int16, np.dtype(np.float16): torch.float16, np.dtype(np.float32): torch.float32}


def _source(a):
    """a quantiser input as the reference passes it -> device array of bf16 bits (uint16) / f16 / f32"""
    if isinstance(a, cp.ndarray):
        return a
    if hasattr(a, "f32"):                        # repo3._Dequant: a quantised seed tensor, dequantised when used
        return a.f32()
    if hasattr(a, "get") and hasattr(a, "into"):     # repo3._Upload: a tensor of a base kept in host memory
        return a.get()
    raise TypeError(f"quantiser input of type {type(a).__name__}")


def to_host(a):
    """device array -> NumPy array in page-locked memory (seedpack/gpuquant.py:262-282)"""
    try:
        host = cp.empty_pinned(a.shape, a.dtype)
    except cp.CUDARuntimeError:
        return a.get()
    a.get(out=host)
    return host


def _download(ys):
    """the tensors of a launch -> one page-locked NumPy array each (a block of its own: the caller may keep it without
    holding the launch's other outputs), copied side by side and waited for once.  The device copy stays registered as
    the array's twin: what the host array is compared with or coded against next is served from it"""
    try:
        hosts = [cp.empty_pinned(y.numel(), np.uint8) for y in ys]
    except cp.CUDARuntimeError:
        return [to_host(from_torch(y)) for y in ys]
    for h, y in zip(hosts, ys):
        torch.from_numpy(h).copy_(y, non_blocking=True)
    torch.cuda.current_stream(ys[0].device).synchronize() if ys else None
    for h, y in zip(hosts, ys):
        cp.STATS["d2h"] += h.nbytes
        twins.register(h, y)
    return hosts


def pcopy(reference_pcopy):
    """repo3._pcopy (repo3.py:516-525: the copy a prediction is cached as, made because a prediction may be a view of
    a launch's whole output): an array that is a page-locked block of its own already is kept as it is"""
    def _pcopy(a):
        r = twins.root(a)
        if cp._PINNED.owns(r) and 8 * a.nbytes >= 7 * r.nbytes:
            return a
        return reference_pcopy(a)
    return _pcopy


def from_torch(t, n=None):
    """a torch uint8 CUDA tensor (kept alive by the array) as a device array of its first n bytes"""
    n = t.numel() if n is None else n
    st = cp._Storage(n)
    st.dev, st.dv = t, True
    return cp.ndarray(st, 0, np.uint8, (n,))


class GPUQuant:
    def __init__(self, fmad=False):
        if fmad:
            raise NotImplementedError("the kernels are built without FMA contraction only (as the archives need)")
        self.q = _gq.GPUQuant(cp.device_index())
        self._imx = {}

    def _imatrix(self, w):
        """importance vectors come as NumPy arrays, the same few objects file after file: uploaded once each"""
        if w is None or isinstance(w, torch.Tensor):
            return w
        if isinstance(w, cp.ndarray):
            return w.dev_in().view(torch.float32)
        w = np.ascontiguousarray(w, np.float32).reshape(-1)
        key = hash(w.tobytes())                      # by content: unit weights are a fresh array per tensor (repo3.py:859-860)
        hit = self._imx.get(key)
        if hit is None or hit[0].size != w.size or not np.array_equal(hit[0], w):
            if len(self._imx) > 4096:
                self._imx.clear()
            hit = (w.copy(), torch.from_numpy(w).to(self.q.device))
            self._imx[key] = hit
        return hit[1]

    def quantize_tensors(self, ttype, srcs, imatrices, variant=0, max_weights=1 << 28, on_result=None, device=False):
        """srcs: [(weights as bf16 bits (uint16) / f16 / f32 device array, or an object that yields one, weights per
        row)] -> the quantised bytes of every tensor: NumPy arrays in page-locked memory, device arrays with `device`;
        with on_result, on_result(index, bytes) per tensor as its group completes, and nothing is returned"""
        cp.device_index()                            # (a worker thread's first call: put it on this process's GPU)
        out, i = [], 0
        while i < len(srcs):
            j, n, group = i, 0, []
            while j < len(srcs) and (j == i or n + srcs[j][0].size <= max_weights):
                a = _source(srcs[j][0])
                if a.dtype not in _TORCH or (group and a.dtype != group[0][0].dtype):
                    if not group:
                        raise TypeError(f"quantiser input of element type {a.dtype}")
                    break
                group.append((a, srcs[j][1])); n += a.size; j += 1
            ts = []
            for a, npr in group:
                t = a.dev_in()
                if t.data_ptr() % 16:               # the kernels load 16 bytes at a time
                    t = t.clone()
                ts.append((t.view(_TORCH[a.dtype]), int(npr)))
            ys = self.q.quantize_tensors(ttype, ts, [self._imatrix(w) for w in imatrices[i:j]], variant, device=True)
            if device:
                res = [from_torch(y) for y in ys]
            else:
                res = _download(ys)
            for k, r in enumerate(res):
                if on_result:
                    on_result(i + k, r)
                else:
                    out.append(r)
            i = j
        return None if on_result else out

    def quantize_batch(self, ttype, xs, imatrices, variant=0):
        """several float32 tensors (nrows, n_per_row) of one type in one launch -> device uint8 arrays"""
        return self.quantize_tensors(ttype, [(x.reshape(-1), x.shape[-1]) for x in xs], imatrices, variant, device=True)

    def dequantize(self, ttype, y, npr, out=None):
        """quantised bytes of a tensor (device uint8) -> float32 device array (or into `out`)"""
        _, qk, bs = QFUN[ttype]
        n = y.size // bs * qk
        x = cp.empty(n, np.float32) if out is None else out
        self.q.dequantize(ttype, y.dev_in(), npr, out=x.dev_out().view(torch.float32))
        return x
