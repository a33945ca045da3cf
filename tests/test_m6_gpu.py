"""M6, the reference's first GPU codec (seedpack/gpu_codec.py: Q8_0 files without a base), on the GPU: the reference's
own M6GPU class runs unmodified over seedpack_b200.refbind, its kernels hist / encode / decode / gather served by
sg_m6_hist / sg_m6_encode / sg_m6_decode / sg_scan_gather.  The compressed file must have the digest the reference's
`--cpu` path gave (tests/golden/m6_digest.json, made by tests/golden/make_m6_golden.py), and decompress to the input."""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "m6_digest.json")))


@pytest.fixture(scope="module")
def codec():
    from seedpack_b200 import refbind
    if not refbind.available():
        pytest.fail("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE)")
    refbind.install()
    from seedpack import gpu_codec
    return gpu_codec


@pytest.fixture(scope="module")
def q8_file(tmp_path_factory):
    from seedpack_b200 import synthrepo
    from test_archive_gpu import gpu_quantizer
    made = synthrepo.make_repo(str(tmp_path_factory.mktemp("m6")), "c1-nano", gpu_quantizer(), seed=GOLD["seed"], only=["Q8_0"])
    return open(made["files"]["Q8_0"], "rb").read()


def test_compressed_file_equals_the_references(codec, q8_file):
    assert [len(q8_file), hashlib.sha256(q8_file).hexdigest()] == GOLD["file"]
    m = codec.M6GPU()
    buf = m.compress(q8_file)
    assert [len(buf), hashlib.sha256(buf).hexdigest()] == GOLD["compressed"]
    assert m.decompress(buf) == q8_file


def test_damaged_stream_is_reported(codec, q8_file):
    m = codec.M6GPU()
    ch = codec.unpack(m.compress(q8_file))
    s = bytearray(ch["stream"])
    s[len(s) // 2] ^= 0x5a
    ch["stream"] = bytes(s)
    with pytest.raises(ValueError, match="corrupt"):
        m.decompress(codec.pack(ch))
