"""llama.cpp quantisers on a B200, bit-identical to ggml-quants.c - host-side mirror of the reference's
`GPUQuant` (seedpack/gpuquant.py:285-456) over the seedgrow C ABI.

Same method names and argument meanings as the reference class: `quantize_tensors`, `quantize_batch`,
`dequantize`; arrays are torch CUDA tensors instead of CuPy arrays.  Differences that follow from
the kernels: BF16 / F16 sources are read directly (no fp32 staging copy, seedpack/gpuquant.py:396-400),
tensors of one launch need not be contiguous with each other (they are addressed by offset from
the lowest address), and a launch has no weight limit.

torch is used for device memory and streams only.
"""
import ctypes

import numpy as np
import torch

from . import _lib
from .requant import NEEDS_IMATRIX, QFUN

_DT = {torch.bfloat16: (_lib.DT_BF16, 2), torch.uint16: (_lib.DT_BF16, 2), torch.int16: (_lib.DT_BF16, 2),
       torch.float16: (_lib.DT_F16, 2), torch.float32: (_lib.DT_F32, 4)}


def _align(n, a):
    return (n + a - 1) // a * a


class GPUQuant:
    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("seedpack_b200 needs a CUDA device: there is no CPU path")
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.lib = _lib.lib()
        self._scratch = None
        self._imx_cache = {}
        from . import tables
        tables.install(self.device.index)

    # ---- helpers ---------------------------------------------------------------------------------
    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _scratch_buf(self, nbytes):
        if nbytes == 0:
            return None, 0
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(_align(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return ctypes.c_void_p(self._scratch.data_ptr()), self._scratch.numel()

    def _imatrix_dev(self, imx):
        if imx is None:
            return None
        if isinstance(imx, torch.Tensor):
            return imx.to(self.device, torch.float32).contiguous().reshape(-1)
        a = np.ascontiguousarray(imx, np.float32).reshape(-1)
        return torch.from_numpy(a).to(self.device)

    def status(self):
        """device status bits set by kernels since the last call (synchronises); 0 = clean"""
        bits = ctypes.c_int(0)
        _lib.check(self.lib.sg_status_fetch(self.device.index, self._stream(), ctypes.byref(bits)), "sg_status_fetch")
        return bits.value

    # ---- the reference's interface ------------------------------------------------------------------
    def quantize_tensors(self, ttype, srcs, imatrices, variant=0, max_weights=None, on_result=None, device=False):
        """srcs: list of (device tensor of the weights as bf16 (bfloat16 / uint16 / int16 bits) / f16 / f32,
        n_per_row).  Returns the quantised bytes of every tensor as numpy arrays (device uint8 tensors
        with `device`), or calls on_result(index, bytes) per tensor and returns None
        (seedpack/gpuquant.py:360-411).  `max_weights` is accepted for compatibility and ignored."""
        if ttype not in QFUN:
            raise ValueError(f"ggml type {ttype} is not a quantised type handled here")
        _, qk, bs = QFUN[ttype]
        if len(srcs) == 0:
            return None if on_result else []
        kinds = {_DT[a.dtype] for a, _ in srcs}
        if len(kinds) != 1:
            raise ValueError("all sources of one launch must have the same element type")
        (dt, esz), = kinds
        tens = (_lib.sg_tensor * len(srcs))()
        base = min(a.data_ptr() for a, _ in srcs)
        ws, wo, yo, spans, keep = [], 0, 0, [], []
        for i, ((a, npr), imx) in enumerate(zip(srcs, imatrices)):
            if not a.is_cuda or not a.is_contiguous():
                raise ValueError("sources must be contiguous CUDA tensors")
            n = a.numel()
            if n % npr or npr % qk:
                raise ValueError(f"tensor {i}: {n} weights do not split into rows of {npr} (block {qk})")
            if imx is None and ttype in NEEDS_IMATRIX:
                raise ValueError(f"ggml type {ttype} needs an importance matrix")
            nr, rb = n // npr, npr // qk * bs
            off = a.data_ptr() - base
            assert off % esz == 0
            tens[i].x_off, tens[i].y_off = off // esz, yo
            tens[i].n_rows, tens[i].n_per_row = nr, npr
            if imx is None:
                tens[i].w_off = -1
            else:
                w = self._imatrix_dev(imx)
                if w.numel() != npr:
                    raise ValueError(f"tensor {i}: importance matrix has {w.numel()} entries for rows of {npr}")
                tens[i].w_off = wo
                ws.append(w); wo += _align(npr, 4)
                if wo != tens[i].w_off + npr:
                    ws.append(torch.zeros(wo - tens[i].w_off - npr, dtype=torch.float32, device=self.device))
            spans.append((yo, nr * rb))
            yo = _align(yo + nr * rb, 16)
            keep.append(a)
        Y = torch.empty(max(yo, 16), dtype=torch.uint8, device=self.device)
        W = torch.cat(ws) if ws else None
        need = self.lib.sg_quantize_scratch_bytes(ttype, tens, len(srcs))
        sp, sn = self._scratch_buf(need)
        rc = self.lib.sg_quantize_tensors(self.device.index, self._stream(), ttype, variant, ctypes.c_void_p(base), dt,
                                          ctypes.c_void_p(Y.data_ptr()), None if W is None else ctypes.c_void_p(W.data_ptr()),
                                          tens, len(srcs), sp, sn)
        _lib.check(rc, f"sg_quantize_tensors(type {ttype})")
        if not device:
            host = torch.empty(Y.shape, dtype=torch.uint8, pin_memory=True)
            host.copy_(Y, non_blocking=False)
            hv = host.numpy()
        out = []
        for i, (o, n) in enumerate(spans):
            r = Y[o:o + n] if device else hv[o:o + n]
            if on_result:
                on_result(i, r)
            else:
                out.append(r)
        return None if on_result else out

    def quantize_batch(self, ttype, xs, imatrices, variant=0):
        """quantise several tensors of one type in one launch.  xs: list of 2-D device tensors
        (nrows, n_per_row); returns device uint8 tensors (seedpack/gpuquant.py:424-430)."""
        return self.quantize_tensors(ttype, [(x.reshape(-1), x.shape[-1]) for x in xs], imatrices, variant, device=True)

    def dequantize(self, ttype, y, npr=None, out=None):
        """quantised bytes of a tensor (device uint8) -> float32 device tensor (or into `out`) with llama.cpp's own
        dequantize_row_<type> (seedpack/gpuquant.py:413-422); `npr` is accepted for compatibility (rows do not matter)"""
        _, qk, bs = QFUN[ttype]
        y = y.view(torch.uint8).reshape(-1)
        n = y.numel() // bs * qk
        x = torch.empty(n, dtype=torch.float32, device=self.device) if out is None else out
        rc = self.lib.sg_dequantize(self.device.index, self._stream(), ttype, ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(x.data_ptr()), n)
        _lib.check(rc, f"sg_dequantize(type {ttype})")
        return x

    def convert_float(self, src, dst_dtype):
        """BF16 / F16 / F32 tensor -> torch.bfloat16 / float16 / float32 (seedpack/repo3.py:673-689 `_float_dev`)"""
        sd = _DT[src.dtype][0]
        dd = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16, torch.float32: _lib.DT_F32}[dst_dtype]
        src = src.contiguous()
        dst = torch.empty(src.numel(), dtype=dst_dtype, device=self.device)
        rc = self.lib.sg_convert_float(self.device.index, self._stream(), ctypes.c_void_p(src.data_ptr()), sd, ctypes.c_void_p(dst.data_ptr()),
                                       dd, src.numel())
        _lib.check(rc, "sg_convert_float")
        return dst
