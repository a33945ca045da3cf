"""Writes tests/golden/quant_extra_golden.npz: the five quantisers of ggml-quants.c that the reference's own type
table leaves out (TQ1_0, TQ2_0, MXFP4, NVFP4, Q1_0), run through the reference's C code as compiled by oracle/Makefile
(oracle/_ref), on a small seeded tensor, with their dequantised values.  Run where the reference tree is mounted (SEEDPACK_REFERENCE names it):

    make -C oracle ref && python tests/golden/make_extra_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref            # noqa: E402
from tests import synth           # noqa: E402

NROWS, NPR = 8, 512
out = {"nrows": NROWS, "npr": NPR}
bits = synth.weights(NROWS, NPR, seed=77)
out["bits"] = bits
x = synth.bf16_bits_to_f32(bits).reshape(NROWS, NPR)
for t in sorted(ref.EXTRA):
    y = ref.quantize(t, x, None, threads=1)
    out[f"q_{t}"] = y
    out[f"d_{t}"] = ref.dequantize(t, y, NROWS * NPR)
np.savez_compressed(os.path.join(HERE, "quant_extra_golden.npz"), **out)
print({k: getattr(v, "shape", v) for k, v in out.items()})
