"""Writes tests/golden/rans_golden.npz with the reference's own coder: seedpack/rans.py (_encode, numba) run per
segment with PROB_BITS = 12 as the GPU coders do (seedpack/qr.py:651-663), tables from the reference's
qr.normalize (seedpack/qr.py:904-923).   python tests/golden/make_rans_golden.py <reference tree>"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import refimport  # noqa: E402

refimport.setup(sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"])
import numpy as np  # noqa: E402
from seedpack import rans as R  # noqa: E402
from seedpack import qr  # noqa: E402

R.PROB_BITS = 12
R.PROB_SCALE = 1 << 12
SEG, BL, NTAB, NSEG = 2048, 32, 7, 5
out = {"seg_len": SEG, "block_len": BL, "ntab": NTAB}
for name, p_zero in (("sparse", 0.97), ("dense", 0.0)):
    rng = np.random.default_rng(12 if name == "sparse" else 13)
    n = SEG * NSEG - 3 * BL                       # last segment is short
    block_tab = rng.integers(0, NTAB, n // BL).astype(np.uint16)
    block_tab[block_tab == 3] = 2                 # table 3 stays unused
    bits = np.array([4, 5, 6, 8, 4, 5, 6])[block_tab]
    lap = np.rint(rng.laplace(0, 2 if name == "sparse" else 6, n)).astype(np.int64)
    sym = np.where(rng.random(n) < p_zero, 0, lap & ((1 << np.repeat(bits, BL)) - 1)).astype(np.uint8)
    ctx = np.repeat(block_tab, BL).astype(np.int32)
    counts = np.bincount(ctx.astype(np.int64) * 256 + sym, minlength=NTAB * 256).reshape(NTAB, 256)
    freq, used = qr.normalize(counts)
    freq, used = np.asarray(freq), np.asarray(used)
    full = np.zeros((NTAB, 256), np.uint16)
    full[used] = freq
    parts, lens = [], []
    for s in range(0, n, SEG):
        b = R.encode(sym[s:s + SEG], ctx[s:s + SEG], full)
        assert np.array_equal(R.decode(b, ctx[s:s + SEG], full), sym[s:s + SEG])
        parts.append(np.frombuffer(b, np.uint8)); lens.append(len(b))
    out.update({f"{name}_sym": sym, f"{name}_block_tab": block_tab, f"{name}_counts": counts, f"{name}_freq": freq,
                f"{name}_used": used, f"{name}_stream": np.concatenate(parts), f"{name}_lens": np.array(lens, np.uint32)})
    print(name, "segments", len(lens), "bytes", sum(lens), "of", n)
np.savez_compressed(os.path.join(HERE, "rans_golden.npz"), **out)
