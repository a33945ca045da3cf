"""Writes tests/golden/qr_seed_golden.npz: coded QR batches made by the REFERENCE (seedpack/qr.py encode, its --cpu
path) with every seed type the kernels read other than plain BF16 - F16 (1), F32 (0), explicit (x, h) pairs (99) and
"no seed" with per-column RMS (98, built by the reference's qr.self_side) - for one scalar-code type (Q4_K) and one
lattice type (IQ2_XS), models 1 and 2.  One tensor is 8192 columns wide, so that every row-position context of model 2
(pos8 / pos4, qr.py:285-286) occurs.
    python tests/golden/make_qr_seed_golden.py <reference tree>"""
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
shapes = [(6, 8192), (16, 1024)]
rng = np.random.default_rng(4242)
out = {"shapes": np.array(shapes)}
xs = [synth.bf16_bits_to_f32(synth.weights(nr, npr, seed=700 + k, edge_cases=False)).reshape(nr, npr) for k, (nr, npr) in enumerate(shapes)]
imxs = [synth.imatrix(npr, seed=800 + k) for k, (_, npr) in enumerate(shapes)]
out["imx"] = np.concatenate(imxs)
imx_offs = [0, shapes[0][1]]


def seeds_of(kind):
    """(seed buffer as uint8, per-tensor byte offsets) for seed type `kind`"""
    parts, offs, o = [], [], 0
    for x in xs:
        if kind == 1:
            a = x.astype(np.float16).view(np.uint8).reshape(-1)
        elif kind == 0:
            a = x.view(np.uint8).reshape(-1)
        else:                                   # 99: (x, h) pairs, h a few per cent of a typical weight
            h = (np.abs(x) * 0.03 + 1e-4).astype(np.float32) * (rng.random(x.shape) < 0.7)
            a = np.stack([x.reshape(-1), h.reshape(-1).astype(np.float32)], 1).reshape(-1).view(np.uint8)
        pad = -len(a) % 256
        parts.append(np.concatenate([a, np.zeros(pad, np.uint8)])); offs.append(o); o += len(a) + pad
    return np.concatenate(parts), offs


for T in (12, 17):
    bs = qr.BS[T]
    use = T in qr.GRID_TYPES
    Fs, Ps = [], []
    for k, x in enumerate(xs):
        w = imxs[k] if use else None
        pred = np.asarray(g.quantize_batch(T, [x], [w])[0]).copy()
        x2 = x.copy()
        rows = rng.random(x.shape[0]) < 0.2
        rows[0] = True
        x2[rows] = x2[rows] * np.float32(1.01) + rng.normal(0, 2e-4, (int(rows.sum()), x.shape[1])).astype(np.float32)
        filed = np.asarray(g.quantize_batch(T, [x2], [w])[0]).copy()
        nb = filed.size // bs
        flip = np.flatnonzero(rng.random(nb) < 0.02)
        filed[flip * bs + rng.integers(0, bs, len(flip))] ^= rng.integers(1, 256, len(flip)).astype(np.uint8)
        Fs.append(filed); Ps.append(pred)
    out[f"F_{T}"], out[f"P_{T}"] = np.concatenate(Fs), np.concatenate(Ps)
    imx_dev = cp.asarray(out["imx"]) if use else None
    for kind in (1, 0, 99):
        seed, offs = seeds_of(kind)
        out[f"seed_{T}_{kind}"], out[f"offs_{T}_{kind}"] = seed, np.array(offs)
        for mv in (1, 2):
            items = [(Fs[k], Ps[k], offs[k], kind, shapes[k][1], imx_offs[k] if use else -1) for k in range(len(xs))]
            buf = qr.encode(T, items, cp.asarray(seed), imx_dev, mv=mv)
            dec = np.asarray(qr.decode(T, buf, [(Ps[k],) + items[k][2:] for k in range(len(xs))], cp.asarray(seed), imx_dev))
            assert np.array_equal(dec, out[f"F_{T}"]), (T, kind, mv)
            out[f"B_{T}_{kind}_{mv}"] = np.frombuffer(buf, np.uint8)
            print("type", T, "seed type", kind, "model", mv, len(buf), "bytes for", out[f"F_{T}"].size)

# no seed (98): the file's own blocks against the template blocks the reference builds from their mean fields
T = 12
Fs98, Ps98, seeds98, offs98, o = [], [], [], [], 0
for k, x in enumerate(xs):
    blocks = cp.asarray(out[f"F_{T}"][sum(len(f) for f in Fs98):][:x.size // 256 * qr.BS[T]])
    rms, tpl, rows = qr.self_side(T, blocks, x.shape[1])
    Fs98.append(np.asarray(blocks)); Ps98.append(np.asarray(cp.tile(tpl, rows)))
    seeds98.append(np.asarray(rms.astype(cp.float32))); offs98.append(o); o += x.shape[1] * 4
out["P98"] = np.concatenate(Ps98)
out["seed98"] = np.concatenate(seeds98).view(np.uint8)
out["offs98"] = np.array(offs98)
for mv in (1, 2):
    items = [(Fs98[k], Ps98[k], offs98[k], 98, shapes[k][1]) for k in range(len(xs))]
    buf = qr.encode(T, items, cp.asarray(out["seed98"]), None, mv=mv)
    dec = np.asarray(qr.decode(T, buf, [(Ps98[k], offs98[k], 98, shapes[k][1]) for k in range(len(xs))], cp.asarray(out["seed98"])))
    assert np.array_equal(dec, out[f"F_{T}"]), ("98", mv)
    out[f"B98_{mv}"] = np.frombuffer(buf, np.uint8)
    print("type", T, "no seed, model", mv, len(buf), "bytes")
np.savez_compressed(os.path.join(HERE, "qr_seed_golden.npz"), **out)
