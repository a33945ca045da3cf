"""Host-side logic that needs no GPU: table normalisation of the base codec, table storage, batch framing, segment
layout, zstd binding - against the reference's own outputs stored in the golden files."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def test_normalize_gpu_matches_reference_tables():
    from seedpack_b200.bf16v2 import normalize_gpu
    from seedpack_b200.qr import load_tables
    G = np.load(os.path.join(HERE, "golden", "r2_golden.npz"))
    freq, used = normalize_gpu(G["counts"], 1 << 15)
    wf, wu = load_tables(G["part_tables"].tobytes())
    assert np.array_equal(used, wu) and np.array_equal(freq, wf)
    assert (freq.astype(np.int64).sum(1) == 1 << 15).all()


def test_store_tables_roundtrip_and_bytes():
    from seedpack_b200.qr import load_tables, store_tables
    G = np.load(os.path.join(HERE, "golden", "r2_golden.npz"))
    buf = G["part_tables"].tobytes()
    freq, used = load_tables(buf)
    assert store_tables(freq, used) == buf                      # same libzstd, same level: same bytes


def test_pack_unpack_and_layout():
    from seedpack_b200 import qr
    G = np.load(os.path.join(HERE, "golden", "qr_golden.npz"))
    buf = G["B_12_2"].tobytes()
    ch = qr.unpack(buf)
    assert list(ch) == ["t", "l", "s", "v"] and bytes(ch["v"]) == b"\x02"
    assert qr.pack({k: bytes(v) for k, v in ch.items()}) == buf
    assert qr.seg_blocks(12) == 64 and qr.seg_blocks(8) == 512 and qr.seg_blocks(42) == 256
    tm, sg, nb = qr._layout(8, [700, 3])
    assert nb == 703 and tm["blk0"].tolist() == [0, 700]
    assert sg.tolist() == [(0, 512, 0), (0, 188, 512), (1, 3, 700)]
    assert qr.batches(12, [200 << 20, 200 << 20, 10]) == [[0], [1, 2]]


def test_zstd_binding_roundtrip():
    from seedpack_b200 import zstd
    data = os.urandom(1000) + bytes(5000)
    for level in (1, 3, 19):
        assert zstd.decompress(zstd.compress(data, level)) == data
    assert zstd.decompress(zstd.compress(b"", 19), 16) == b""


def test_imatrix_loader(tmp_path):
    import struct
    from seedpack_b200.requant import imatrix_chunks, load_imatrix
    vals = np.arange(8, dtype=np.float32)
    name = b"blk.0.ffn_up.weight"
    buf = struct.pack("<i", 1) + struct.pack("<i", len(name)) + name + struct.pack("<ii", 4, 8) + vals.tobytes() + struct.pack("<i", 77)
    d = load_imatrix(buf)
    assert np.array_equal(d["blk.0.ffn_up.weight"], vals / 4)
    assert imatrix_chunks(buf) == 77
