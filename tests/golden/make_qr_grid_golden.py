"""Writes tests/golden/qr_grid_golden.npz: coded QR batches of the lattice (IQ) types made by the REFERENCE
(seedpack/qr.py encode, --cpu path), models 1 and 2, with an importance matrix, on small seeded tensors.
    python tests/golden/make_qr_grid_golden.py <reference tree>"""
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
TYPES = [16, 17, 18, 19, 21, 22, 29]
shapes = [(20, 512), (10, 1024)]
out = {"types": np.array(TYPES), "shapes": np.array(shapes)}
rng = np.random.default_rng(7)
seed_bits, offs, imxs, ioffs, o, io = [], [], [], [], 0, 0
for k, (nr, npr) in enumerate(shapes):
    b = synth.weights(nr, npr, seed=700 + k)
    seed_bits.append(b.reshape(-1)); offs.append(o * 2); o += b.size
    imxs.append(synth.imatrix(npr, seed=40 + k)); ioffs.append(io); io += npr
seed = np.concatenate(seed_bits)
imx = np.concatenate(imxs)
out.update(seed_bits=seed, seed_offs=np.array(offs), imx=imx, imx_offs=np.array(ioffs))
for T in TYPES:
    bs = qr.BS[T]
    items_f, items_p = [], []
    for k, (nr, npr) in enumerate(shapes):
        x = synth.bf16_bits_to_f32(seed_bits[k]).reshape(nr, npr)
        pred = np.asarray(g.quantize_batch(T, [x], [imxs[k]])[0]).copy()
        x2 = x.copy()
        rows = rng.random(nr) < 0.1
        rows[1] = True
        x2[rows] = x2[rows] * np.float32(1.02) + rng.normal(0, 5e-4, (int(rows.sum()), npr)).astype(np.float32)
        filed = np.asarray(g.quantize_batch(T, [x2], [imxs[k]])[0]).copy()
        nb = filed.size // bs
        flip = np.flatnonzero(rng.random(nb) < 0.05)
        filed[flip * bs + rng.integers(2, bs, len(flip))] ^= rng.integers(1, 256, len(flip)).astype(np.uint8)
        items_f.append(filed); items_p.append(pred)
    out[f"F_{T}"] = np.concatenate(items_f); out[f"P_{T}"] = np.concatenate(items_p)
    for mv in (1, 2):
        items = [(items_f[k], items_p[k], offs[k], 30, shapes[k][1], ioffs[k]) for k in range(len(shapes))]
        buf = qr.encode(T, items, seed.view(np.uint8), imx, mv=mv)
        dec = np.asarray(qr.decode(T, buf, [(items_p[k], offs[k], 30, shapes[k][1], ioffs[k]) for k in range(len(shapes))],
                                   seed.view(np.uint8), imx))
        assert np.array_equal(dec, out[f"F_{T}"]), (T, mv)
        out[f"B_{T}_{mv}"] = np.frombuffer(buf, np.uint8)
        print(T, mv, len(buf), "bytes for", out[f"F_{T}"].size, "ne blocks",
              int((out[f"F_{T}"].reshape(-1, bs) != out[f"P_{T}"].reshape(-1, bs)).any(1).sum()), flush=True)
np.savez_compressed(os.path.join(HERE, "qr_grid_golden.npz"), **out)
