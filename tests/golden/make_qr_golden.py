"""Writes tests/golden/qr_golden.npz: coded QR batches made by the REFERENCE (seedpack/qr.py encode, its --cpu path) for
every scalar-code type, models 1 and 2: stored file blocks = the reference quantiser's output (no importance matrix)
of a perturbed copy of the weights plus byte flips, predictions = its output on the seed weights.
    python tests/golden/make_qr_golden.py <reference tree>"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import refimport  # noqa: E402

refimport.setup(sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"])
import numpy as np  # noqa: E402
from seedpack import gpuquant, qr  # noqa: E402
from tests import synth  # noqa: E402

g = gpuquant.GPUQuant()
TYPES = [2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 20, 23, 42]
shapes = [(40, 512), (24, 768)]             # two tensors per batch; > 1 segment each for the 32-weight block types
out = {"types": np.array(TYPES), "shapes": np.array(shapes)}
rng = np.random.default_rng(99)
seed_bits, offs, o = [], [], 0
for k, (nr, npr) in enumerate(shapes):
    b = synth.weights(nr, npr, seed=300 + k)
    seed_bits.append(b.reshape(-1)); offs.append(o * 2); o += b.size
seed = np.concatenate(seed_bits)
out["seed_bits"] = seed
out["seed_offs"] = np.array(offs)
for T in TYPES:
    bs = qr.BS[T]
    items_f, items_p = [], []
    for k, (nr, npr) in enumerate(shapes):
        x = synth.bf16_bits_to_f32(seed_bits[k]).reshape(nr, npr)
        pred = np.asarray(g.quantize_batch(T, [x], [None])[0]).copy()
        # the stored file: same quantiser on slightly different weights in 3 % of the rows (scales and codes move), plus
        # single-byte flips in 0.5 % of the blocks
        x2 = x.copy()
        rows = rng.random(nr) < 0.03
        rows[0] = True
        x2[rows] = x2[rows] * np.float32(1.01) + rng.normal(0, 2e-4, (int(rows.sum()), npr)).astype(np.float32)
        filed = np.asarray(g.quantize_batch(T, [x2], [None])[0]).copy()
        nb = filed.size // bs
        flip = np.flatnonzero(rng.random(nb) < 0.005)
        filed[flip * bs + rng.integers(0, bs, len(flip))] ^= rng.integers(1, 256, len(flip)).astype(np.uint8)
        items_f.append(filed); items_p.append(pred)
    out[f"F_{T}"] = np.concatenate(items_f); out[f"P_{T}"] = np.concatenate(items_p)
    for mv in (1, 2):
        items = [(items_f[k], items_p[k], offs[k], 30, shapes[k][1], -1) for k in range(len(shapes))]
        buf = qr.encode(T, items, seed.view(np.uint8), None, mv=mv)
        dec = np.asarray(qr.decode(T, buf, [(items_p[k], offs[k], 30, shapes[k][1], -1) for k in range(len(shapes))], seed.view(np.uint8)))
        assert np.array_equal(dec, out[f"F_{T}"]), (T, mv)
        out[f"B_{T}_{mv}"] = np.frombuffer(buf, np.uint8)
        print(T, mv, len(buf), "bytes for", out[f"F_{T}"].size, "ne blocks", int((out[f"F_{T}"].reshape(-1, bs) != out[f"P_{T}"].reshape(-1, bs)).any(1).sum()))
np.savez_compressed(os.path.join(HERE, "qr_golden.npz"), **out)
