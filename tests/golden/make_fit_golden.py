"""Writes tests/golden/fit_golden.npz: outputs of the reference's remaining detmath kernels (dm_rows_d, dm_gram, dm_bdot,
dm_solve; seedpack/detmath.py:86-153) from its --cpu path, on seeded inputs.
    python tests/golden/make_fit_golden.py <reference tree>"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import refimport  # noqa: E402

refimport.setup(sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"])
import numpy as np  # noqa: E402
from seedpack import detmath  # noqa: E402

rng = np.random.default_rng(77)
out = {}
out["rows_x"] = (rng.standard_normal((19, 301)) * np.exp(rng.normal(0, 3, (19, 301)))).astype(np.float64)
out["rows"] = np.asarray(detmath.rows(out["rows_x"]))
out["rows_sq"] = np.asarray(detmath.rows(out["rows_x"], True))
X = (rng.standard_normal((5, 7, 257)) * np.exp(rng.normal(0, 2, (5, 7, 257)))).astype(np.float32)
y = rng.standard_normal((5, 257)).astype(np.float32)
out["X"], out["y"] = X, y
out["gram"] = np.asarray(detmath.gram(X))
out["bdot"] = np.asarray(detmath.bdot(X, y))
for k in (1, 3, 16):
    A = rng.standard_normal((11, k, k)).astype(np.float32)
    A[3] = 0                                        # a singular system: whatever comes out must be the same bits
    A[5, 0, 0] = 0                                  # needs a row exchange
    b = rng.standard_normal((11, k)).astype(np.float32)
    out[f"A{k}"], out[f"b{k}"] = A, b
    with np.errstate(all="ignore"):
        out[f"x{k}"] = np.asarray(detmath.solve(A, b))
np.savez_compressed(os.path.join(HERE, "fit_golden.npz"), **out)
print({k: v.shape for k, v in out.items()})
