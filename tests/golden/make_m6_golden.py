"""Writes tests/golden/m6_digest.json from the REFERENCE's --cpu path: the Q8_0 file of the seeded repository "c1-nano"
(seedpack_b200.synthrepo, quantised by the reference's C code) compressed by seedpack/gpu_codec.py's M6GPU - size and
SHA-256 of the file and of the compressed bytes.
    python tests/golden/make_m6_golden.py <reference tree>"""
import hashlib
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import refimport  # noqa: E402

refimport.setup(sys.argv[1] if len(sys.argv) > 1 else os.environ["SEEDPACK_REFERENCE"])
from oracle import ref  # noqa: E402
from seedpack import gpu_codec  # noqa: E402
from seedpack_b200 import synthrepo  # noqa: E402

SEED = 1
with tempfile.TemporaryDirectory() as tmp:
    made = synthrepo.make_repo(tmp, "c1-nano", lambda ty, bits, w: ref.quantize(ty, ref.bf16_to_f32(bits), w), seed=SEED, only=["Q8_0"])
    data = open(made["files"]["Q8_0"], "rb").read()
m = gpu_codec.M6GPU()
buf = m.compress(data)
assert m.decompress(buf) == data
sha = lambda b: hashlib.sha256(b).hexdigest()
out = {"seed": SEED, "file": [len(data), sha(data)], "compressed": [len(buf), sha(buf)]}
json.dump(out, open(os.path.join(HERE, "m6_digest.json"), "w"), indent=1)
print(out)
