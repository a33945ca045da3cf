"""Writes tests/golden/iq_table_digests.json from the reference's seedpack/ggml/iqtables.npz (run where the
reference tree is mounted):  python tests/golden/make_table_digests.py <reference tree>"""
import hashlib
import json
import os
import sys

import numpy as np

ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"]
tb = np.load(os.path.join(ref, "seedpack", "ggml", "iqtables.npz"))
names = ["iq2_data_0", "iq2_data_1", "iq2_data_2", "iq2_data_3", "iq3_data_0", "iq3_data_1"]
out = {}
for i, n in enumerate(names):
    for k in ("grid", "map", "nb"):
        a = np.ascontiguousarray(tb[f"{n}_{k}"])
        out[f"{i}_{k}"] = {"n": int(a.size), "dtype": str(a.dtype), "sha256": hashlib.sha256(a.tobytes()).hexdigest()}
json.dump(out, open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "iq_table_digests.json"), "w"), indent=1)
