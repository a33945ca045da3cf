"""The detmath kernels behind the importance fit (sg_dm_rows_f64, sg_dm_gram, sg_dm_bdot, sg_dm_solve) against the
reference's outputs (tests/golden/fit_golden.npz, made by tests/golden/make_fit_golden.py from its --cpu path): bit for
bit, NaNs of a singular system included."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fit_golden.npz"))


def _call(name, *args):
    import torch
    from seedpack_b200 import _lib
    conv = [ctypes.c_void_p(a.data_ptr()) if isinstance(a, torch.Tensor) else a for a in args]
    rc = getattr(_lib.lib(), name)(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), *conv)
    _lib.check(rc, name)


def _same_bits(a, b):
    u = {4: np.uint32, 8: np.uint64}[a.dtype.itemsize]
    return np.array_equal(np.ascontiguousarray(a).view(u), np.ascontiguousarray(b).view(u))


def test_rows_of_a_float64_matrix():
    import torch
    x = torch.from_numpy(G["rows_x"]).cuda()
    for sq, key in ((0, "rows"), (1, "rows_sq")):
        out = torch.empty(x.shape[0], dtype=torch.float64, device="cuda")
        _call("sg_dm_rows_f64", x, x.shape[0], x.shape[1], sq, out)
        assert _same_bits(out.cpu().numpy(), G[key]), key


def test_gram_and_products():
    import torch
    X, y = torch.from_numpy(G["X"]).cuda(), torch.from_numpy(G["y"]).cuda()
    nb, k, d = X.shape
    g = torch.empty((nb, k, k), dtype=torch.float32, device="cuda")
    _call("sg_dm_gram", X, nb, k, d, g)
    assert _same_bits(g.cpu().numpy(), G["gram"])
    p = torch.empty((nb, k), dtype=torch.float32, device="cuda")
    _call("sg_dm_bdot", X, y, nb, k, d, p)
    assert _same_bits(p.cpu().numpy(), G["bdot"])


@pytest.mark.parametrize("k", [1, 3, 16])
def test_small_systems(k):
    import torch
    A, b = torch.from_numpy(G[f"A{k}"]).cuda(), torch.from_numpy(G[f"b{k}"]).cuda()
    x = torch.empty_like(b)
    _call("sg_dm_solve", A, b, A.shape[0], k, x)
    got, want = x.cpu().numpy(), G[f"x{k}"]
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert _same_bits(np.where(nan, 0, got).astype(np.float32), np.where(nan, 0, want).astype(np.float32))


def test_more_than_16_unknowns_is_refused():
    import torch
    from seedpack_b200 import _lib
    A = torch.zeros((1, 17, 17), device="cuda"); b = torch.zeros((1, 17), device="cuda")
    rc = _lib.lib().sg_dm_solve(0, None, ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(b.data_ptr()), 1, 17, ctypes.c_void_p(b.data_ptr()))
    assert rc == 11                                   # SG_ERR_LIMIT
