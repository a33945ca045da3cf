"""The reference's older codecs for files without a base, on the GPU, through its own unmodified classes over
seedpack_b200.refbind:
  * M6 (seedpack/gpu_codec.py, Q8_0 files): kernels hist / encode / decode / gather served by sg_m6_hist / sg_m6_encode /
    sg_m6_decode / sg_scan_gather;
  * M22 (seedpack/bf16codec.py, BF16 files): rans.encode / rans.decode (seedpack/rans.py, one rANS state per stream, 14
    probability bits) served by sg_rans_chain_encode / sg_rans_chain_decode.
The compressed files must have the digests the reference's `--cpu` path gave (tests/golden/legacy_codec_digests.json,
made by tests/golden/make_legacy_codec_golden.py), and decompress to their inputs."""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "legacy_codec_digests.json")))


@pytest.fixture(scope="module")
def ref():
    from seedpack_b200 import refbind
    if not refbind.available():
        pytest.fail("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE)")
    refbind.install()
    from seedpack import bf16codec, gpu_codec, rans
    return gpu_codec, bf16codec, rans


@pytest.fixture(scope="module")
def files(tmp_path_factory):
    from seedpack_b200 import synthrepo
    from tests.test_archive_gpu import gpu_quantizer
    made = synthrepo.make_repo(str(tmp_path_factory.mktemp("legacy")), "c1-nano", gpu_quantizer(), seed=GOLD["seed"], only=["Q8_0"])
    return open(made["files"]["Q8_0"], "rb").read(), open(made["base"][0], "rb").read()


def _sig(b):
    return [len(b), hashlib.sha256(b).hexdigest()]


def test_m6_compressed_file_equals_the_references(ref, files):
    q8 = files[0]
    assert _sig(q8) == GOLD["m6"]["file"]
    m = ref[0].M6GPU()
    buf = m.compress(q8)
    assert _sig(buf) == GOLD["m6"]["compressed"]
    assert bytes(m.decompress(buf)) == q8


def test_m6_damaged_stream_is_reported(ref, files):
    codec = ref[0]
    m = codec.M6GPU()
    ch = dict(codec.unpack(m.compress(files[0])))
    s = bytearray(ch["stream"])
    s[len(s) // 2] ^= 0x5a
    ch["stream"] = bytes(s)
    with pytest.raises(ValueError, match="corrupt"):
        m.decompress(codec.pack(ch))


def test_m22_compressed_file_equals_the_references(ref, files):
    bf = files[1]
    assert _sig(bf) == GOLD["m22"]["file"]
    m = ref[1].M22BF16()
    buf = m.compress(bf)
    assert _sig(buf) == GOLD["m22"]["compressed"]
    assert bytes(m.decompress(buf)) == bf


def test_scalar_coder_edges(ref):
    """rans.encode / rans.decode over the chain kernels: an empty stream is the four state bytes; int32 contexts; a
    context outside the tables and a symbol without frequency are refused on the host / reported by the kernel"""
    rans = ref[2]
    rng = np.random.default_rng(5)
    ctx = rng.integers(0, 7, 5000).astype(np.int32)
    sym = np.minimum(rng.geometric(0.3, 5000) + ctx, 255).astype(np.uint8)
    f = rans.build_freqs(sym, ctx, 7)
    buf = rans.encode(sym, ctx, f)
    assert np.array_equal(rans.decode(buf, ctx, f), sym)
    assert rans.encode(sym[:0], ctx[:0], f) == b"\x00\x80\x00\x00"
    with pytest.raises(ValueError, match="context"):
        rans.encode(sym, ctx + 3, f)
    g = f.copy()
    s0, c0 = int(sym[0]), int(ctx[0])
    other = int(np.argmax(g[c0] * (np.arange(256) != s0)))
    g[c0, other] += g[c0, s0]; g[c0, s0] = 0
    with pytest.raises(ValueError, match="frequency 0"):
        rans.encode(sym, ctx, g)
