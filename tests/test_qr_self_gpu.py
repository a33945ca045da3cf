"""Coding without a BF16 seed (tests/golden/qr_self_golden.npz, made by the reference's --cpu path): sibling quants as
seeds (the seed buffer holds Q8_0 / Q6_K / IQ4_XS blocks; value = dequantised weight, uncertainty = half a code step),
self-coding from column statistics and template blocks (qr.self_encode: the reference's own function over the bound
block_fields / blocks_from_fields / dequantiser / detmath / coder kernels), and the helper kernels."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_self_golden.npz"))
SHAPES = [tuple(int(v) for v in s) for s in G["shapes"]]


def _items(T, ST):
    from seedpack_b200.qr import BS, GRID_TYPES, QK
    F, P, bs = G[f"F_{T}"], G[f"P_{T}"], BS[T]
    enc, dec, o, io = [], [], 0, 0
    for k, (nr, npr) in enumerate(SHAPES):
        n = nr * npr // QK[T] * bs
        tail = (int(G[f"offs_{ST}"][k]), ST, npr, io if T in GRID_TYPES else -1)
        enc.append((F[o:o + n], P[o:o + n]) + tail); dec.append((P[o:o + n],) + tail)
        o += n; io += npr
    return enc, dec


@pytest.mark.parametrize("ST", [8, 14, 23])
@pytest.mark.parametrize("T", [12, 17])
def test_quantised_seeds_match_the_reference(T, ST):
    from seedpack_b200.qr import GRID_TYPES, QRCodec
    c = QRCodec()
    enc, dec = _items(T, ST)
    seed, imx = G[f"seed_{ST}"], (G["imx"] if T in GRID_TYPES else None)
    want = G[f"B_{T}_{ST}"].tobytes()
    for staged in (True, False):
        c.staged = staged
        assert c.encode(T, enc, seed, imx, mv=2) == want, f"staged={staged}"
    assert np.array_equal(c.decode(T, want, dec, seed, imx).cpu().numpy(), G[f"F_{T}"])


def _call(name, *args):
    import torch
    from seedpack_b200 import _lib
    conv = [ctypes.c_void_p(a.data_ptr()) if isinstance(a, torch.Tensor) else a for a in args]
    _lib.check(getattr(_lib.lib(), name)(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), *conv), name)


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def test_helper_kernels_match_the_reference():
    import torch
    from seedpack_b200 import tables
    tables.install(0)
    nw = sum(nr * nc for nr, nc in SHAPES)
    F, P = torch.from_numpy(G["F_12"]).cuda(), torch.from_numpy(G["P_12"]).cuda()
    lo, hi = torch.empty(nw, device="cuda"), torch.empty(nw, device="cuda")
    _call("sg_qr_intervals", 12, F, nw, lo, hi)
    assert np.array_equal(_bits(lo.cpu().numpy()), _bits(G["lo_12"])) and np.array_equal(_bits(hi.cpu().numpy()), _bits(G["hi_12"]))
    n23 = SHAPES[0][0] * SHAPES[0][1]
    S = torch.from_numpy(G["seed_23"][:n23 // 256 * 136].copy()).cuda()
    lo, hi = torch.empty(n23, device="cuda"), torch.empty(n23, device="cuda")
    _call("sg_qr_intervals", 23, S, n23, lo, hi)
    assert np.array_equal(_bits(lo.cpu().numpy()), _bits(G["lo_23"])) and np.array_equal(_bits(hi.cpu().numpy()), _bits(G["hi_23"]))
    eq = torch.empty(nw, dtype=torch.uint8, device="cuda")
    _call("sg_qr_weight_equal", 12, F, P, nw, eq)
    assert np.array_equal(eq.cpu().numpy(), G["weq_12"])
    F17 = torch.from_numpy(G["F_17"]).cuda()
    h = torch.empty(nw, device="cuda")
    _call("sg_qr_grid_half_step", 17, F17, nw, h)
    assert np.array_equal(_bits(h.cpu().numpy()), _bits(G["gridh_17"]))
    nblk = nw // 256
    fl = torch.empty(nblk * 18, dtype=torch.int32, device="cuda")
    _call("sg_qr_block_fields", 12, F, nblk, fl)
    assert np.array_equal(fl.cpu().numpy(), G["fields_12"])
    back = torch.empty(nblk * 144, dtype=torch.uint8, device="cuda")
    _call("sg_qr_blocks_from_fields", 12, fl, nblk, back)           # the fields again, codes zero
    fl2 = torch.empty_like(fl)
    _call("sg_qr_block_fields", 12, back, nblk, fl2)
    assert torch.equal(fl, fl2) and int(back.view(-1, 144)[:, 16:].sum()) == 0


def test_self_coding_through_the_references_own_function():
    """qr.self_encode / self_decode of the reference, unmodified, over the bound kernels"""
    from seedpack_b200 import refbind
    if not refbind.available():
        pytest.fail("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE)")
    refbind.install()
    from seedpack import qr
    n0 = SHAPES[0][0] * SHAPES[0][1] // 256 * 144
    tens = [(G["F_12"][:n0], SHAPES[0][1]), (G["F_12"][n0:], SHAPES[1][1])]
    buf = qr.self_encode(12, tens)
    assert bytes(buf) == G["self_12"].tobytes()
    back = qr.self_decode(12, G["self_12"].tobytes())
    for b, t in zip(back, tens):
        assert np.array_equal(b.get(), t[0])
