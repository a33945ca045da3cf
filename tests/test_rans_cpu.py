"""CPU checks of the rANS checker and of the host-side table normalisation against golden vectors made with the
reference's own coder (tests/golden/make_rans_golden.py: seedpack/rans.py per segment at 12 probability bits,
tables from seedpack/qr.py normalize)."""
import os

import numpy as np
import pytest

from oracle import rans as orans

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rans_golden.npz"))
SEG, BL, NTAB = int(G["seg_len"]), int(G["block_len"]), int(G["ntab"])


def _full(name):
    full = np.zeros((NTAB, 256), np.uint16)
    full[G[f"{name}_used"]] = G[f"{name}_freq"]
    return full


@pytest.mark.parametrize("name", ["sparse", "dense"])
def test_normalize_matches_reference(name):
    from seedpack_b200.rans import normalize
    f, u = normalize(G[f"{name}_counts"])
    assert np.array_equal(f, G[f"{name}_freq"]) and np.array_equal(u, G[f"{name}_used"])
    assert (f.astype(np.int64).sum(1) == 4096).all()


def test_normalize_edge_rows():
    from seedpack_b200.rans import normalize
    c = np.zeros((4, 256), np.int64)
    c[0, 7] = 5                                  # one symbol: takes the whole range
    c[1, :] = 1                                  # 256 equally rare symbols
    c[2, 0] = 10 ** 9; c[2, 1:] = 1              # one dominant symbol and 255 rare ones (each must keep 1)
    f, u = normalize(c)
    assert u.tolist() == [0, 1, 2] and f[0, 7] == 4096 and (f[1] == 16).all()
    assert f[2, 0] == 4096 - 255 and (f[2, 1:] == 1).all()


@pytest.mark.parametrize("name", ["sparse", "dense"])
def test_port_encode_matches_golden(name):
    stream, off = orans.encode(G[f"{name}_sym"], G[f"{name}_block_tab"], BL, SEG, _full(name))
    assert np.array_equal(np.diff(off).astype(np.uint32), G[f"{name}_lens"])
    assert np.array_equal(stream, G[f"{name}_stream"])
    out, rc = orans.decode(stream, off, G[f"{name}_block_tab"], BL, len(G[f"{name}_sym"]), SEG, _full(name))
    assert rc == 0 and np.array_equal(out, G[f"{name}_sym"])


def test_port_decode_flags_truncation():
    name = "dense"
    stream, off = orans.encode(G[f"{name}_sym"], G[f"{name}_block_tab"], BL, SEG, _full(name))
    off2 = off.copy(); off2[-1] -= 3
    _, rc = orans.decode(stream, off2, G[f"{name}_block_tab"], BL, len(G[f"{name}_sym"]), SEG, _full(name))
    assert rc == 1
