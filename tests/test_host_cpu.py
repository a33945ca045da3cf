"""Host-side logic that needs no GPU: table normalisation of the base codec, table storage, batch framing, segment
layout, zstd binding - against the reference's own outputs stored in the golden files."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def test_normalize_gpu_matches_reference_tables():
    """the reference's own gpu2.normalize_gpu, run over the binding's array module (host-resident arrays: NumPy arithmetic,
    stable sorts; no device is touched), gives the tables its --cpu run stored"""
    import subprocess
    import sys
    from seedpack_b200 import refbind
    from seedpack_b200.qr import load_tables
    ref = refbind.find_reference()
    if ref is None:
        import pytest
        pytest.skip("needs the reference package (baseline/_ref or $SEEDPACK_REFERENCE)")
    code = (
        "import sys, importlib.util, numpy as np\n"
        f"sys.path[:0] = [{os.path.dirname(HERE)!r}, {ref!r}]\n"
        "from seedpack_b200.refbind import cupy_shim as cp\n"
        "sys.modules['cupy'], sys.modules['cupyx'] = cp, cp.cupyx\n"
        "if importlib.util.find_spec('zstandard') is None:\n"
        "    from seedpack_b200 import zstd; sys.modules['zstandard'] = zstd\n"
        "from seedpack import gpu2\n"
        f"G = np.load({os.path.join(HERE, 'golden', 'r2_golden.npz')!r})\n"
        "f, u = gpu2.normalize_gpu(cp._wrap(np.ascontiguousarray(G['counts'])), 1 << 15)\n"
        "np.save(sys.argv[1], f.get()); np.save(sys.argv[2], u.get())\n"
        "assert cp.STATS['h2d'] == 0 and cp.STATS['d2h'] == 0\n")
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        a, b = os.path.join(tmp, "f.npy"), os.path.join(tmp, "u.npy")
        env = {k: v for k, v in os.environ.items() if k != "SEEDPACK_CPU"}
        r = subprocess.run([sys.executable, "-c", code, a, b], capture_output=True, text=True, env=env, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        freq, used = np.load(a), np.load(b)
    G = np.load(os.path.join(HERE, "golden", "r2_golden.npz"))
    wf, wu = load_tables(G["part_tables"].tobytes(), 15)
    assert np.array_equal(used, wu) and np.array_equal(freq, wf)
    assert (freq.astype(np.int64).sum(1) == 1 << 15).all()


def test_store_tables_roundtrip_and_bytes():
    from seedpack_b200.qr import load_tables, store_tables
    G = np.load(os.path.join(HERE, "golden", "r2_golden.npz"))
    buf = G["part_tables"].tobytes()
    freq, used = load_tables(buf, 15)
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


def test_zstd_streams_and_prefix_dictionary():
    """the parts of the zstandard interface the archive layer uses: streamed compression with a pledged size and worker
    threads, a raw-content dictionary, and the forward reader"""
    import io
    from seedpack_b200 import zstd
    rng = np.random.default_rng(5)
    head = rng.integers(0, 256, 4096, np.uint8).tobytes()
    data = head * 3 + bytes(200000) + rng.integers(0, 4, 300000, np.uint8).tobytes()
    zd = zstd.ZstdCompressionDict(head, dict_type=zstd.DICT_TYPE_RAWCONTENT)
    prm = zstd.ZstdCompressionParameters.from_level(7, window_log=25, threads=4)
    whole = zstd.ZstdCompressor(compression_params=prm, dict_data=zd).compress(data)
    assert zstd.ZstdDecompressor(dict_data=zd).decompress(whole) == data
    obj = zstd.ZstdCompressor(compression_params=prm, dict_data=zd).compressobj(size=len(data))
    parts = [obj.compress(data[o:o + 70001]) for o in range(0, len(data), 70001)] + [obj.flush()]
    frame = b"".join(parts)
    out = bytearray(len(data))
    with zstd.ZstdDecompressor(dict_data=zd).stream_reader(io.BytesIO(frame), read_size=1 << 12) as r:
        o = 0
        while o < len(out):
            k = r.readinto(memoryview(out)[o:o + 50000])
            assert k
            o += k
    assert bytes(out) == data
    with zstd.ZstdDecompressor(dict_data=zd).stream_reader(frame) as r:
        assert r.read() == data
    plain = zstd.ZstdCompressor(level=19).compress(data)
    assert len(whole) < len(plain)           # the dictionary removes the three copies of `head`


def test_damaged_table_part_is_rejected_before_any_launch():
    """a `t` part whose rows do not sum to 2^PB (or whose ids run backwards) never reaches sg_rans_tables"""
    import struct
    import pytest
    from seedpack_b200 import zstd
    from seedpack_b200.qr import check_lens, check_tables, load_tables, store_tables
    freq = np.zeros((2, 256), np.uint16)
    freq[0, 0], freq[0, 7] = 4000, 96
    freq[1, 3] = 4096
    good = store_tables(freq, np.array([5, 90]))
    f, u = load_tables(good, 12, 294)
    assert np.array_equal(f, freq) and list(u) == [5, 90]
    bad = freq.copy(); bad[1, 3] = 65535; bad[1, 4] = 65535          # sums far beyond 2^12
    with pytest.raises(ValueError):
        load_tables(store_tables(bad, np.array([5, 90])), 12, 294)
    with pytest.raises(ValueError):
        load_tables(store_tables(freq, np.array([5, 400])), 12, 294)  # id beyond the table count
    raw = struct.pack("<I", 2) + struct.pack("<II", 9, 0) + freq.tobytes()
    with pytest.raises(ValueError):
        load_tables(zstd.compress(raw, 3), 12, 294)                   # ids not increasing
    with pytest.raises(ValueError):
        load_tables(zstd.compress(raw[:-10], 3), 12, 294)             # truncated
    counts = np.zeros((294, 256), np.int64)
    counts[5, 0] = 10; counts[90, 3] = 1
    check_tables(freq, [5, 90], counts)
    counts[5, 9] = 1                                                  # occurs, but the table gives it nothing
    with pytest.raises(ValueError):
        check_tables(freq, [5, 90], counts)
    with pytest.raises(ValueError):
        check_lens(np.array([10, 0xfffffffe], np.uint32))


def test_batch_records_are_bounds_checked_on_the_host():
    """offsets into the seed and importance buffers, and the seed type, are checked before any launch"""
    import pytest
    from seedpack_b200.qr import check_records
    T = 12                                            # Q4_K: 256 weights per block
    ok = dict(T=T, nblocks=[8, 4], seed_offs=[0, 4096], seed_types=[30, 30], cols=[1024, 1024], imx_offs=[-1, -1],
              seed_bytes=4096 + 4 * 256 * 2, imx_floats=0)
    check_records(**ok)
    for change in (dict(seed_bytes=4096 + 4 * 256 * 2 - 2),            # the last tensor's seed runs past the buffer
                   dict(seed_offs=[0, -2]), dict(seed_offs=[1, 4096]),  # negative / odd BF16 offset
                   dict(seed_types=[30, 17]),                           # a lattice type cannot be a seed
                   dict(seed_types=[30, 77]),
                   dict(seed_types=[30, 8], seed_offs=[0, 5200]),       # a Q8_0 seed whose blocks run past the buffer
                   dict(cols=[1000, 1024]),                             # not whole blocks per row
                   dict(cols=[1024, 768]),                              # 4 blocks are not whole rows of 768
                   dict(imx_offs=[0, -1], imx_floats=1000),             # importance vector shorter than a row
                   dict(imx_offs=[-3, -1])):
        with pytest.raises(ValueError):
            check_records(**{**ok, **change})
    check_records(T, [8], [0], [98], [1024], [-1], 4096, 0)          # no seed: one float per column
    with pytest.raises(ValueError):
        check_records(T, [8], [0], [98], [0], [-1], 4096, 0)         # ... needs the row length
    check_records(17, [8], [0], [0], [2048], [0], 8 * 256 * 4, 2048)  # F32 seed, lattice type with importance values
    check_records(T, [8], [0], [99], [0], [-1], 8 * 256 * 8, 0)       # explicit (x, h) pairs
    check_records(T, [8], [0], [8], [1024], [-1], 8 * 256 // 32 * 34, 0)   # a sibling Q8_0 tensor as the seed
