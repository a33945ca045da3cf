"""Writes tests/golden/legacy_codec_digests.json from the REFERENCE's --cpu path, on files of the seeded repository
"c1-nano" (seedpack_b200.synthrepo, quantised by the reference's C code):
  m6   the Q8_0 file compressed by seedpack/gpu_codec.py's M6GPU,
  m22  the BF16 file compressed by seedpack/bf16codec.py's M22BF16 (the scalar coder of seedpack/rans.py),
each with size and SHA-256 of the file and of the compressed bytes.
    python tests/golden/make_legacy_codec_golden.py <reference tree>"""
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
from seedpack import bf16codec, gpu_codec  # noqa: E402
from seedpack_b200 import synthrepo  # noqa: E402

SEED = 1
sha = lambda b: hashlib.sha256(b).hexdigest()
with tempfile.TemporaryDirectory() as tmp:
    made = synthrepo.make_repo(tmp, "c1-nano", lambda ty, bits, w: ref.quantize(ty, ref.bf16_to_f32(bits), w), seed=SEED, only=["Q8_0"])
    q8 = open(made["files"]["Q8_0"], "rb").read()
    bf = open(made["base"][0], "rb").read()
out = {"seed": SEED}
for key, codec, data in (("m6", gpu_codec.M6GPU(), q8), ("m22", bf16codec.M22BF16(), bf)):
    buf = codec.compress(data)
    assert bytes(codec.decompress(buf)) == data
    out[key] = {"file": [len(data), sha(data)], "compressed": [len(buf), sha(buf)]}
    print(key, out[key])
json.dump(out, open(os.path.join(HERE, "legacy_codec_digests.json"), "w"), indent=1)
