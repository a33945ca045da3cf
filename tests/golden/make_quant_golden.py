"""Writes tests/golden/quant_golden.npz: outputs of the REFERENCE ITSELF (its --cpu path: the kernels of
seedpack/gpuquant.py compiled for the host by seedpack/cpukernels.py) for every quantised type, with and
without an importance matrix, plus the IQ1_M variant, on a small seeded tensor.  Run where the reference
tree is mounted:

    python tests/golden/make_quant_golden.py <reference tree>

The fixture holds its own inputs (bf16 bit patterns and the importance matrix), so no test needs the
reference tree."""
import os
import sys

ref_tree = sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"]
os.environ["SEEDPACK_CPU"] = "1"
os.environ.setdefault("SEEDPACK_CACHE", "/tmp/seedpack-golden-cache")
os.makedirs(os.environ["SEEDPACK_CACHE"], exist_ok=True)
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ref_tree)
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import numpy as np  # noqa: E402
from seedpack import gpuquant  # noqa: E402  (the reference package)
from seedpack.requant import QFUN  # noqa: E402
from tests import synth  # noqa: E402

NROWS, NPR = 12, 768
bits = synth.weights(NROWS, NPR, seed=2024)
imx = synth.imatrix(NPR, seed=2024)
x = synth.bf16_bits_to_f32(bits).reshape(NROWS, NPR)
g = gpuquant.GPUQuant()
out = {"bits": bits, "imatrix": imx}
needs = {16, 17, 19}
for t in sorted(QFUN):
    for use in ((True,) if t in needs else (True, False)):
        y = np.asarray(g.quantize_batch(t, [x], [imx if use else None])[0])
        out[f"t{t}_{'imx' if use else 'none'}_v0"] = y.copy()
for use in (True, False):
    y = np.asarray(g.quantize_batch(29, [x], [imx if use else None], variant=1)[0])
    out[f"t29_{'imx' if use else 'none'}_v1"] = y.copy()
np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), **out)
print("cases:", len(out) - 2, "bytes:", sum(v.nbytes for v in out.values()))
