"""R2 BF16 base codec and detmath through the C ABI against parts coded by the reference's own BF16v2.compress
(tests/golden/r2_golden.npz, written by tests/golden/make_r2_golden.py): side information, tables, segment lengths and
stream must be byte-identical; decoding the reference's parts must restore every tensor."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "r2_golden.npz"))


def _parts():
    return {k[5:]: G[k].tobytes() for k in G.files if k.startswith("part_")}


def _layout():
    from seedpack_b200 import zstd
    return json.loads(zstd.decompress(_parts()["meta"], 1 << 20))


def test_compress_parts_are_byte_identical_to_reference():
    from seedpack_b200 import zstd
    from seedpack_b200.bf16v2 import BF16v2
    meta = _layout()
    got = BF16v2(group_bytes=150_000).compress_parts(G["data"], meta["layout"])
    want = _parts()
    gm = json.loads(zstd.decompress(got["meta"], 1 << 20))
    assert gm == meta                                            # layout, duplicate rows, compact row counts
    for k in ("side", "tables", "lens"):
        assert zstd.decompress(got[k], 1 << 30) == zstd.decompress(want[k], 1 << 30), k
    assert got["stream"] == want["stream"]
    for k in ("meta", "side", "tables", "lens"):
        assert got[k] == want[k], f"{k}: same content but different zstd framing"


def test_decode_of_reference_parts_restores_tensors():
    from seedpack_b200.bf16v2 import R2Tensors
    r = R2Tensors(_parts())
    t = r.layout["t"]
    dev, outs = r.decode(range(len(t)))
    h = dev.cpu().numpy()
    for k, (off, nb, rl, _) in enumerate(t):
        assert np.array_equal(h[outs[k]:outs[k] + nb], G["data"][off:off + nb]), k
    dev, outs = r.decode([3, 0])                                  # random access, any order
    h = dev.cpu().numpy()
    for k, i in enumerate([3, 0]):
        off, nb = t[i][0], t[i][1]
        assert np.array_equal(h[outs[k]:outs[k] + nb], G["data"][off:off + nb])


def test_group_size_does_not_change_the_bytes_of_the_tables():
    """the group split changes the stream's grouping only: counts (hence tables) are sums over the whole file"""
    from seedpack_b200.bf16v2 import BF16v2
    meta = _layout()
    a = BF16v2(group_bytes=150_000).compress_parts(G["data"], meta["layout"])
    b = BF16v2(group_bytes=1 << 30).compress_parts(G["data"], meta["layout"])
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
