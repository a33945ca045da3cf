"""The allocation-free entry point, sg_quantize_legacy_imx_static, against sg_quantize_tensors.

It exists for hosts that cannot let the library allocate device memory while they run (a packer whose windows
already account for every free byte; a pipeline that cannot afford cudaMalloc's device-wide stall) and that
have no pool to lend scratch from: its per-row scratch is a fixed array inside the library.  Both entry points
must give the same bytes (the quantisers are bit-exact, so the tolerance is zero), on two calls in a row -
the second call finds the first call's contents in the shared array.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest

from tests import synth

pytestmark = pytest.mark.gpu


def _run(L, fn_static, t, x, w, y, tens, n, dev, stream, scratch):
    if fn_static:
        return L.sg_quantize_legacy_imx_static(dev, stream, t, ctypes.c_void_p(x.data_ptr()), 0, ctypes.c_void_p(y.data_ptr()),
                                               ctypes.c_void_p(w.data_ptr()), tens, n)
    return L.sg_quantize_tensors(dev, stream, t, 0, ctypes.c_void_p(x.data_ptr()), 0, ctypes.c_void_p(y.data_ptr()),
                                 ctypes.c_void_p(w.data_ptr()), tens, n, ctypes.c_void_p(scratch.data_ptr()), scratch.numel())


def test_static_scratch_entry_matches_regular_entry():
    import torch
    from seedpack_b200 import _lib
    L = _lib.lib()
    dev = torch.cuda.current_device()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    shapes = [(40, 1024), (7, 288)]
    for call in range(2):                                    # two calls in a row, different data each time
        for t, bs in ((2, 18), (3, 20), (6, 22), (7, 24)):
            xs, ws, tens, xo, yo, wo = [], [], (_lib.sg_tensor * len(shapes))(), 0, 0, 0
            for k, (nr, npr) in enumerate(shapes):
                xs.append(synth.weights(nr, npr, seed=900 + 10 * call + k, edge_cases=False).reshape(-1))
                ws.append(synth.imatrix(npr, seed=call + k))
                tens[k].x_off, tens[k].y_off, tens[k].w_off, tens[k].n_rows, tens[k].n_per_row = xo, yo, wo, nr, npr
                xo += nr * npr; yo += (nr * npr // 32 * bs + 15) // 16 * 16; wo += npr
            x = torch.from_numpy(np.concatenate(xs).view(np.int16)).cuda()
            w = torch.from_numpy(np.concatenate(ws)).cuda()
            ya = torch.zeros(yo, dtype=torch.uint8, device="cuda")
            yb = torch.zeros(yo, dtype=torch.uint8, device="cuda")
            scratch = torch.empty(4096, dtype=torch.uint8, device="cuda")
            assert _run(L, False, t, x, w, ya, tens, len(shapes), dev, stream, scratch) == 0
            assert _run(L, True, t, x, w, yb, tens, len(shapes), dev, stream, scratch) == 0
            torch.cuda.synchronize()
            assert torch.equal(ya, yb), f"type {t}, call {call}"
            assert int(ya.count_nonzero()) > 0


def test_static_scratch_entry_rejects_what_it_cannot_hold():
    import torch
    from seedpack_b200 import _lib
    L = _lib.lib()
    dev = torch.cuda.current_device()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = ctypes.c_void_p(buf.data_ptr())
    t = (_lib.sg_tensor * 1)()
    t[0].x_off, t[0].y_off, t[0].w_off, t[0].n_rows, t[0].n_per_row = 0, 0, 0, 65537, 32
    assert L.sg_quantize_legacy_imx_static(dev, None, 2, p, 0, p, p, t, 1) == 11          # SG_ERR_LIMIT: too many rows
    t[0].n_rows, t[0].w_off = 4, -1
    assert L.sg_quantize_legacy_imx_static(dev, None, 2, p, 0, p, p, t, 1) == 5           # needs an importance matrix
    t[0].w_off = 0
    assert L.sg_quantize_legacy_imx_static(dev, None, 12, p, 0, p, p, t, 1) == 2          # not a type that uses scratch
