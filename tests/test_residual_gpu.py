"""Residual kernels against NumPy (the reference computes these on the host with NumPy, seedpack/repo3.py:456-510)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _pair(n, seed, frac=0.005):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, n, dtype=np.uint8)
    b = a.copy()
    k = max(1, int(n * frac))
    idx = rng.choice(n, k, replace=False)
    b[idx] ^= rng.integers(1, 256, k, dtype=np.uint8)
    return a, b


@pytest.mark.parametrize("n,off", [(0, 0), (1, 0), (15, 0), (16, 0), (4097, 0), (1 << 20, 0), ((1 << 20) + 7, 3), (34 * 999, 2)])
def test_xor_and_counts(n, off):
    import torch
    from seedpack_b200 import residual
    a, b = _pair(n + off, 1) if n + off else (np.zeros(0, np.uint8), np.zeros(0, np.uint8))
    c = np.random.default_rng(2).integers(0, 256, n + off, dtype=np.uint8)
    ta, tb, tc = (torch.from_numpy(v).cuda()[off:] for v in (a, b, c))      # off makes the pointers unaligned
    a, b, c = a[off:], b[off:], c[off:]
    if n == 0:
        return
    assert residual.count_diff(ta, tb) == int(np.count_nonzero(a != b))
    assert residual.count_diff(ta) == int(np.count_nonzero(a))
    o, k = residual.xor3(ta, tb, tc)
    assert np.array_equal(o.cpu().numpy(), a ^ b ^ c) and k == int(np.count_nonzero(a ^ b ^ c))
    r = ta.clone()
    left = residual.xor_(r, tb)
    assert np.array_equal(r.cpu().numpy(), a ^ b) and left == int(np.count_nonzero(a ^ b))
    assert residual.xor_(tb.clone(), tb) == 0                                # exact prediction: nothing left


@pytest.mark.parametrize("bs", [18, 34, 66, 110, 144, 210])
def test_block_flags(bs):
    import torch
    from seedpack_b200 import residual
    nb = 5000
    a, b = _pair(nb * bs, bs, frac=0.001)
    ne, cnt = residual.block_ne(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), bs)
    want = (a.reshape(nb, bs) != b.reshape(nb, bs)).any(axis=1)
    assert np.array_equal(ne.cpu().numpy().astype(bool), want) and cnt == int(want.sum())


def test_quantise_then_residual_roundtrip():
    """prediction == stored file except for flipped bytes: the residual is exactly the flips, and XOR-ing it back
    restores the file (the bijection unpack relies on)"""
    import torch
    from seedpack_b200 import residual
    from seedpack_b200.gpuquant import GPUQuant
    from tests import synth
    gq = GPUQuant()
    bits = synth.weights(64, 2048, seed=9)
    x = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16).reshape(-1)
    pred = gq.quantize_tensors(12, [(x, 2048)], [None], device=True)[0]
    stored = pred.clone()
    rng = np.random.default_rng(0)
    pos = torch.from_numpy(rng.choice(stored.numel(), 37, replace=False)).cuda()
    stored[pos] ^= 0x5a
    res = stored.clone()
    assert residual.xor_(res, pred) == 37
    back = res.clone()
    assert residual.xor_(back, pred) >= 0 and torch.equal(back, stored)
