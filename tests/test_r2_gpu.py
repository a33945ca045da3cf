"""R2 BF16 base codec and detmath on the GPU against parts coded by the reference's own BF16v2.compress
(tests/golden/r2_golden.npz, written by tests/golden/make_r2_golden.py).  The host side IS the reference's: its
BF16v2 / R2Tensors classes (seedpack/bf16v2.py:174-617) run unmodified over seedpack_b200.refbind, so what is compared
is the reference's framing around this library's kernels (sg_r2_stats, sg_row_hash, sg_r2_hist / encode / decode,
sg_scan_gather, sg_rans_tables): every part of the coded file must be byte-identical, and decoding the reference's
parts must restore every tensor."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "r2_golden.npz"))


def _parts():
    return {k[5:]: G[k].tobytes() for k in G.files if k.startswith("part_")}


@pytest.fixture(scope="module")
def ref():
    from seedpack_b200 import refbind
    if not refbind.available():
        pytest.fail("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE)")
    refbind.install()
    from seedpack import bf16v2, codecs_gguf
    return bf16v2, codecs_gguf


def _compress(ref, group_bytes):
    bf16v2, codecs_gguf = ref
    parts = bf16v2.BF16v2(group_bytes=group_bytes).compress_parts(G["data"].tobytes())
    return {k: bytes(v) for k, v in codecs_gguf.unpack(b"".join(bytes(p) for p in parts)).items()}


def test_compress_parts_are_byte_identical_to_reference(ref):
    got, want = _compress(ref, 150_000), _parts()
    for k in ("meta", "side", "tables", "lens", "stream"):
        assert got[k] == want[k], k
    assert set(got) == set(want) | {"rest"}


def test_decode_of_reference_parts_restores_tensors(ref):
    bf16v2, _ = ref
    want = _parts()
    got = _compress(ref, 150_000)                                  # (the golden file keeps no `rest` part: ours is the same function's)
    parts = dict(want, rest=got["rest"])
    stream = np.frombuffer(parts["stream"], np.uint8)

    def read(o, n, out):
        np.frombuffer(out, np.uint8)[:n] = stream[o:o + n]
        return out

    r = bf16v2.R2Tensors(lambda name: parts[name], read)
    t = r.layout["t"]
    dev, outs = r.decode(range(len(t)))
    h = dev.get()
    for k, (off, nb, rl, _) in enumerate(t):
        assert np.array_equal(h[outs[k]:outs[k] + nb], G["data"][off:off + nb]), k
    dev, outs = r.decode([3, 0])                                  # random access, any order
    h = dev.get()
    for k, i in enumerate([3, 0]):
        off, nb = t[i][0], t[i][1]
        assert np.array_equal(h[outs[k]:outs[k] + nb], G["data"][off:off + nb])
    whole = bf16v2.BF16v2().decompress(ref[1].pack(parts))
    assert np.array_equal(np.asarray(whole), G["data"])


def test_group_size_does_not_change_the_bytes_of_the_tables(ref):
    """the group split changes the stream's grouping only: counts (hence tables) are sums over the whole file"""
    a, b = _compress(ref, 150_000), _compress(ref, 1 << 30)
    assert a["tables"] == b["tables"] and a["side"] == b["side"] and a["stream"] == b["stream"]


def test_detmath_matches_reference_bits():
    import torch
    from seedpack_b200 import detmath
    x = torch.from_numpy(G["dm_x"]).cuda()
    assert np.array_equal(detmath.log2(x).cpu().numpy().view(np.uint64), G["dm_log2"].view(np.uint64))
    y = torch.from_numpy(G["dm_y"]).cuda()
    assert np.array_equal(detmath.exp2(y).cpu().numpy().view(np.uint64), G["dm_exp2"].view(np.uint64))
    m = torch.from_numpy(G["dm_m"]).cuda()
    for fn, sq, key in ((detmath.rows, False, "dm_rows"), (detmath.rows, True, "dm_rows_sq"), (detmath.cols, False, "dm_cols"),
                        (detmath.cols, True, "dm_cols_sq")):
        assert np.array_equal(fn(m, sq).cpu().numpy().view(np.uint64), G[key].view(np.uint64)), key
