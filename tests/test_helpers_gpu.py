"""The device forms of the three helpers every quantiser leans on, over their whole input range.

  * float32 -> float16 bits (the integer / float construction of ggml-impl.h:417-443), all 2^32 inputs, through
    sg_convert_float, against the hardware's round-to-nearest-even conversion; NaN inputs must give the canonical
    sign | 0x7e00 the C code gives;
  * float16 -> float32 (ggml-impl.h:396-415), all 2^16 inputs, against the hardware conversion, bit for bit;
  * BF16 rounding of float32 (the integer add of seedpack/repo3.py:687-688), 2^28 inputs spread over the range, against
    that formula in integers;
  * nearest_int (ggml-quants.c:621-626: add 1.5 * 2^23, read the mantissa) through sg_selftest_nearest_int over a dense
    sweep of the range the C code asserts (|x| <= 4194303) against round-half-to-even, and out-of-range inputs against
    the C expression evaluated in integers.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
DT_BF16, DT_F16, DT_F32 = 0, 1, 2


def _convert(src, sd, dst, dd, n):
    import torch
    from seedpack_b200 import _lib
    rc = _lib.lib().sg_convert_float(torch.cuda.current_device(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                     ctypes.c_void_p(src.data_ptr()), sd, ctypes.c_void_p(dst.data_ptr()), dd, n)
    _lib.check(rc, "sg_convert_float")


def test_f32_to_f16_all_inputs():
    import torch
    n = 1 << 26
    out = torch.empty(n, dtype=torch.int16, device="cuda")
    for chunk in range(64):
        bits = torch.arange(chunk * n, (chunk + 1) * n, dtype=torch.int64, device="cuda").to(torch.int32)      # wraps into all 2^32 patterns
        x = bits.view(torch.float32)
        _convert(x, DT_F32, out, DT_F16, n)
        want = x.to(torch.float16).view(torch.int16)
        nan = torch.isnan(x)
        canon = (((bits >> 16) & 0x8000) | 0x7e00).to(torch.int16)
        want = torch.where(nan, canon, want)
        bad = int((out != want).sum())
        assert bad == 0, f"chunk {chunk}: {bad} inputs differ"


def test_f16_to_f32_all_inputs():
    import torch
    h = torch.arange(0, 1 << 16, dtype=torch.int32, device="cuda").to(torch.int16)
    out = torch.empty(1 << 16, dtype=torch.float32, device="cuda")
    _convert(h, DT_F16, out, DT_F32, 1 << 16)
    want = h.view(torch.float16).to(torch.float32)
    a, b = out.view(torch.int32), want.view(torch.int32)
    nan = torch.isnan(want)
    assert bool(((a == b) | nan).all())
    assert bool(torch.isnan(out)[nan].all())


def test_f32_to_bf16_rounding():
    import torch
    n = 1 << 28
    bits = (torch.arange(0, n, dtype=torch.int64, device="cuda") * 16 + 5).to(torch.int32)
    out = torch.empty(n, dtype=torch.int16, device="cuda")
    _convert(bits.view(torch.float32), DT_F32, out, DT_BF16, n)
    u = bits.to(torch.int64) & 0xffffffff
    want = ((u + 0x7fff + ((u >> 16) & 1)) >> 16) & 0xffff
    assert bool((out.to(torch.int64) & 0xffff == want).all())


def test_nearest_int_dense_sweep():
    import torch
    from seedpack_b200 import _lib
    L = _lib.lib()
    n = 1 << 26
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    for scale in (1.0, 40.0, 4000.0, 4194303.0):
        x = (torch.rand(n, generator=g, device="cuda", dtype=torch.float64) * 2 - 1).mul_(scale).to(torch.float32)
        x[:9] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.0, -0.0, scale], device="cuda")
        _lib.check(L.sg_selftest_nearest_int(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(x.data_ptr()),
                                             ctypes.c_void_p(out.data_ptr()), n), "sg_selftest_nearest_int")
        want = torch.round(x.to(torch.float64)).to(torch.int32)          # half to even, as the magic-number add rounds
        assert bool((out == want).all()), scale
    # outside the asserted range the C expression still has a value: (bits(x + 12582912.f) & 0x7fffff) - 0x400000
    # (NaN is left out: the sum is a NaN on both sides, but its payload is the processor's choice)
    x = torch.tensor([5e6, -5e6, 1e9, -3e7, float("inf"), -float("inf")], device="cuda", dtype=torch.float32)
    o = torch.empty(6, dtype=torch.int32, device="cuda")
    _lib.check(L.sg_selftest_nearest_int(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(x.data_ptr()),
                                         ctypes.c_void_p(o.data_ptr()), 6), "sg_selftest_nearest_int")
    v = (x.cpu().numpy() + np.float32(12582912.0)).astype(np.float32).view(np.int32)
    assert o.cpu().numpy().tolist() == ((v & 0x7fffff) - 0x400000).tolist()
