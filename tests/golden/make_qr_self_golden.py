"""Writes tests/golden/qr_self_golden.npz, from the REFERENCE's --cpu path (seedpack/qr.py):
  * coded batches whose seed is a sibling QUANT (seed types 8 Q8_0, 14 Q6_K, 23 IQ4_XS; qr.py:331-344) for targets
    Q4_K (12) and IQ2_XS (17), model 2;
  * qr.self_encode of two Q4_K tensors (no seed: block_fields, blocks_from_fields, column RMS; qr.py:1116-1152);
  * outputs of the helper kernels intervals / weq / grid_h / block_fields on those blocks (qr.py:985-1005, 811-878).
    python tests/golden/make_qr_self_golden.py <reference tree>"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import refimport  # noqa: E402

refimport.setup(sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"])
import numpy as np  # noqa: E402
from seedpack import gpuquant, qr  # noqa: E402
from seedpack.xp import cp  # noqa: E402
from tests import synth  # noqa: E402

g = gpuquant.GPUQuant()
shapes = [(8, 2048), (16, 1024)]
rng = np.random.default_rng(99)
out = {"shapes": np.array(shapes)}
xs = [synth.bf16_bits_to_f32(synth.weights(nr, npr, seed=900 + k, edge_cases=False)).reshape(nr, npr) for k, (nr, npr) in enumerate(shapes)]
imxs = [synth.imatrix(npr, seed=950 + k) for k, (_, npr) in enumerate(shapes)]
out["imx"] = np.concatenate(imxs)
imx_offs = [0, shapes[0][1]]
quant = lambda T, x, w=None: np.asarray(g.quantize_batch(T, [x], [w])[0]).copy()

for T in (12, 17):
    use = T in qr.GRID_TYPES
    bs = qr.BS[T]
    Fs, Ps = [], []
    for k, x in enumerate(xs):
        w = imxs[k] if use else None
        Ps.append(quant(T, x, w))
        x2 = x * np.float32(1.004) + rng.normal(0, 1e-4, x.shape).astype(np.float32)
        f = quant(T, x2, w)
        nb = f.size // bs
        flip = np.flatnonzero(rng.random(nb) < 0.03)
        f[flip * bs + rng.integers(0, bs, len(flip))] ^= rng.integers(1, 256, len(flip)).astype(np.uint8)
        Fs.append(f)
    out[f"F_{T}"], out[f"P_{T}"] = np.concatenate(Fs), np.concatenate(Ps)
    imx_dev = cp.asarray(out["imx"]) if use else None
    for ST in (8, 14, 23):
        seeds, offs, o = [], [], 0
        for x in xs:
            s = quant(ST, x, None)
            pad = -len(s) % 256
            seeds.append(np.concatenate([s, np.zeros(pad, np.uint8)])); offs.append(o); o += len(s) + pad
        seed = np.concatenate(seeds)
        out[f"seed_{ST}"], out[f"offs_{ST}"] = seed, np.array(offs)
        items = [(Fs[k], Ps[k], offs[k], ST, shapes[k][1], imx_offs[k] if use else -1) for k in range(len(xs))]
        buf = qr.encode(T, items, cp.asarray(seed), imx_dev, mv=2)
        dec = np.asarray(qr.decode(T, buf, [(Ps[k],) + items[k][2:] for k in range(len(xs))], cp.asarray(seed), imx_dev))
        assert np.array_equal(dec, out[f"F_{T}"]), (T, ST)
        out[f"B_{T}_{ST}"] = np.frombuffer(buf, np.uint8)
        print("target", T, "seed quant", ST, len(buf), "bytes")

T = 12
tens = [(out["F_12"][:xs[0].size // 256 * 144], shapes[0][1]), (out["F_12"][xs[0].size // 256 * 144:], shapes[1][1])]
buf = qr.self_encode(T, tens)
back = qr.self_decode(T, buf)
assert all(np.array_equal(np.asarray(b), t[0]) for b, t in zip(back, tens))
out["self_12"] = np.frombuffer(buf, np.uint8)
print("self_encode", len(buf), "bytes")
nw = sum(x.size for x in xs)
lo, hi = qr.intervals(12, cp.asarray(out["F_12"]), nw)
out["lo_12"], out["hi_12"] = np.asarray(lo), np.asarray(hi)
lo, hi = qr.intervals(23, cp.asarray(out["seed_23"][:xs[0].size // 256 * 136]), xs[0].size)
out["lo_23"], out["hi_23"] = np.asarray(lo), np.asarray(hi)
out["weq_12"] = np.asarray(qr.weight_equal(12, cp.asarray(out["F_12"]), cp.asarray(out["P_12"]), nw))
h = cp.empty(nw, cp.float32)
qr.kern("grid_h")(((nw + 255) // 256,), (256,), (np.int32(17), cp.asarray(out["F_17"]), np.int64(nw), h))
out["gridh_17"] = np.asarray(h)
nblk = nw // 256
fl = cp.empty(nblk * qr.NFIELDS[12], cp.int32)
qr.kern("block_fields")(((nblk + 255) // 256,), (256,), (np.int32(12), cp.asarray(out["F_12"]), np.int64(nblk), fl))
out["fields_12"] = np.asarray(fl)
np.savez_compressed(os.path.join(HERE, "qr_self_golden.npz"), **out)
