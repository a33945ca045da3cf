"""QR residual coder through the C ABI against coded batches made by the reference's own qr.encode
(tests/golden/qr_golden.npz, written by tests/golden/make_qr_golden.py): the whole packed batch - tables, segment
lengths, stream, model byte - must be byte-identical, and decoding the reference's batch must restore the file."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_golden.npz"))
TYPES = [int(t) for t in G["types"]]
SHAPES = [tuple(int(v) for v in s) for s in G["shapes"]]
OFFS = [int(o) for o in G["seed_offs"]]


def _items(T):
    from seedpack_b200.qr import BS
    F, P, bs = G[f"F_{T}"], G[f"P_{T}"], BS[T]
    from seedpack_b200.qr import QK
    enc, dec, o = [], [], 0
    for k, (nr, npr) in enumerate(SHAPES):
        n = nr * npr // QK[T] * bs
        enc.append((F[o:o + n], P[o:o + n], OFFS[k], 30, npr, -1))
        dec.append((P[o:o + n], OFFS[k], 30, npr, -1))
        o += n
    return enc, dec


@pytest.mark.parametrize("mv", [1, 2])
@pytest.mark.parametrize("T", TYPES)
def test_encode_is_byte_identical_to_reference(T, mv):
    from seedpack_b200.qr import QRCodec, unpack
    c = QRCodec()
    enc, _ = _items(T)
    got = c.encode(T, enc, G["seed_bits"].view(np.uint8), None, mv=mv)
    want = G[f"B_{T}_{mv}"].tobytes()
    if got != want:
        a, b = unpack(got), unpack(want)
        diff = {k: (len(a.get(k, b"")), len(b.get(k, b"")), bytes(a.get(k, b"")) == bytes(b.get(k, b""))) for k in set(a) | set(b)}
        raise AssertionError(f"type {T} model {mv}: parts (ours, reference, equal) = {diff}")


@pytest.mark.parametrize("mv", [1, 2])
@pytest.mark.parametrize("T", TYPES)
def test_decode_of_reference_batch_restores_file(T, mv):
    from seedpack_b200.qr import QRCodec
    c = QRCodec()
    _, dec = _items(T)
    out = c.decode(T, G[f"B_{T}_{mv}"].tobytes(), dec, G["seed_bits"].view(np.uint8))
    assert np.array_equal(out.cpu().numpy(), G[f"F_{T}"])


def test_exact_prediction_codes_to_flags_only():
    """a file equal to its prediction: one flag symbol per block, every other table unused"""
    from seedpack_b200.qr import QRCodec, unpack, load_tables
    c = QRCodec()
    T = 12
    enc, dec = _items(T)
    same = [(it[1], it[1]) + it[2:] for it in enc]
    buf = c.encode(T, same, G["seed_bits"].view(np.uint8))
    freq, used = load_tables(unpack(buf)["t"])
    assert used.tolist() == [85] and freq[0, 1] == 4096          # FLAG + prev = 1, symbol "equal"
    out = c.decode(T, buf, dec, G["seed_bits"].view(np.uint8))
    assert np.array_equal(out.cpu().numpy(), G[f"P_{T}"])


def test_corrupt_batch_is_rejected():
    from seedpack_b200.qr import QRCodec, unpack, pack
    c = QRCodec()
    _, dec = _items(8)
    ch = {k: bytes(v) for k, v in unpack(G["B_8_2"].tobytes()).items()}
    s = bytearray(ch["s"]); s[len(s) // 2] ^= 0x40; ch["s"] = bytes(s)
    try:
        out = c.decode(8, pack(ch), dec, G["seed_bits"].view(np.uint8))
    except ValueError:
        return
    assert not np.array_equal(out.cpu().numpy(), G["F_8"])


# ---- lattice (IQ) types ---------------------------------------------------------------------------------------------
GG = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_grid_golden.npz"))
GTYPES = [int(t) for t in GG["types"]]
GSHAPES = [tuple(int(v) for v in s) for s in GG["shapes"]]


def _grid_items(T):
    from seedpack_b200.qr import BS
    F, P, bs = GG[f"F_{T}"], GG[f"P_{T}"], BS[T]
    enc, dec, o = [], [], 0
    for k, (nr, npr) in enumerate(GSHAPES):
        n = nr * npr // 256 * bs
        so, io = int(GG["seed_offs"][k]), int(GG["imx_offs"][k])
        enc.append((F[o:o + n], P[o:o + n], so, 30, npr, io))
        dec.append((P[o:o + n], so, 30, npr, io))
        o += n
    return enc, dec


@pytest.mark.parametrize("mv", [1, 2])
@pytest.mark.parametrize("T", GTYPES)
def test_grid_encode_is_byte_identical_to_reference(T, mv):
    from seedpack_b200.qr import QRCodec, unpack
    c = QRCodec()
    enc, _ = _grid_items(T)
    got = c.encode(T, enc, GG["seed_bits"].view(np.uint8), GG["imx"], mv=mv)
    want = GG[f"B_{T}_{mv}"].tobytes()
    if got != want:
        a, b = unpack(got), unpack(want)
        diff = {k: (len(a.get(k, b"")), len(b.get(k, b"")), bytes(a.get(k, b"")) == bytes(b.get(k, b""))) for k in set(a) | set(b)}
        raise AssertionError(f"type {T} model {mv}: parts (ours, reference, equal) = {diff}")


@pytest.mark.parametrize("mv", [1, 2])
@pytest.mark.parametrize("T", GTYPES)
def test_grid_decode_of_reference_batch_restores_file(T, mv):
    from seedpack_b200.qr import QRCodec
    c = QRCodec()
    _, dec = _grid_items(T)
    out = c.decode(T, GG[f"B_{T}_{mv}"].tobytes(), dec, GG["seed_bits"].view(np.uint8), GG["imx"])
    assert np.array_equal(out.cpu().numpy(), GG[f"F_{T}"])


@pytest.mark.parametrize("T", TYPES)
def test_single_pass_and_staged_encoders_agree(T):
    """sg_qr_hist + sg_qr_encode (one lane per segment) and sg_qr_stage* (one lane per block, then the coder) give the
    same batch"""
    from seedpack_b200.qr import QRCodec
    enc, _ = _items(T)
    seed = G["seed_bits"].view(np.uint8)
    assert QRCodec(staged=False).encode(T, enc, seed, None, mv=2) == QRCodec(staged=True).encode(T, enc, seed, None, mv=2)


@pytest.mark.parametrize("T", GTYPES)
def test_grid_single_pass_and_staged_encoders_agree(T):
    from seedpack_b200.qr import QRCodec
    enc, _ = _grid_items(T)
    seed = GG["seed_bits"].view(np.uint8)
    assert QRCodec(staged=False).encode(T, enc, seed, GG["imx"], mv=2) == QRCodec(staged=True).encode(T, enc, seed, GG["imx"], mv=2)


# ---- seed types other than BF16, wide rows (tests/golden/qr_seed_golden.npz, made by the reference) -----------------------
GS = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_seed_golden.npz"))
S_SHAPES = [tuple(int(v) for v in s) for s in GS["shapes"]]


def _seed_items(T, kind):
    from seedpack_b200.qr import BS, GRID_TYPES, QK
    F, P, bs = GS[f"F_{T}"], (GS["P98"] if kind == 98 else GS[f"P_{T}"]), BS[T]
    offs = GS["offs98"] if kind == 98 else GS[f"offs_{T}_{kind}"]
    enc, dec, o, io = [], [], 0, 0
    for k, (nr, npr) in enumerate(S_SHAPES):
        n = nr * npr // QK[T] * bs
        tail = (int(offs[k]), kind, npr, io if T in GRID_TYPES else -1)
        enc.append((F[o:o + n], P[o:o + n]) + tail)
        dec.append((P[o:o + n],) + tail)
        o += n; io += npr
    return enc, dec


@pytest.mark.parametrize("mv", [1, 2])
@pytest.mark.parametrize("T,kind", [(12, 1), (12, 0), (12, 99), (12, 98), (17, 1), (17, 0), (17, 99)])
def test_other_seed_types_match_the_reference(T, kind, mv):
    """F16, F32, explicit (x, h) and column-RMS seeds; an 8192-column tensor reaches every row-position context"""
    from seedpack_b200.qr import GRID_TYPES, QRCodec
    c = QRCodec()
    enc, dec = _seed_items(T, kind)
    seed = GS["seed98"] if kind == 98 else GS[f"seed_{T}_{kind}"]
    imx = GS["imx"] if T in GRID_TYPES else None
    want = (GS[f"B98_{mv}"] if kind == 98 else GS[f"B_{T}_{kind}_{mv}"]).tobytes()
    for staged in (True, False):
        c.staged = staged
        assert c.encode(T, enc, seed, imx, mv=mv) == want, f"staged={staged}"
    assert np.array_equal(c.decode(T, want, dec, seed, imx).cpu().numpy(), GS[f"F_{T}"])


def test_unknown_seed_type_is_refused():
    from seedpack_b200.qr import QRCodec
    enc, _ = _seed_items(12, 1)
    bad = [it[:3] + (17,) + it[4:] for it in enc]            # a lattice type cannot stand in for the seed
    with pytest.raises(ValueError):
        QRCodec().encode(12, bad, GS["seed_12_1"], None)


# ---- sharded coding: segment ranges, counts summed before the tables are made ------------------------------------------------
@pytest.mark.parametrize("T", [8, 12, 17])
def test_batch_coded_in_segment_ranges_equals_the_references_batch(T):
    """what every rank of a sharded run does, here one range after the other on one GPU: model and count a range of
    segments, add the counts, normalise once, code each range, join lengths and bytes in segment order"""
    from seedpack_b200 import shard
    from seedpack_b200.qr import MODEL, QRCodec, _layout, BS
    from seedpack_b200.rans import normalize
    c = QRCodec()
    if T == 17:
        G2 = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qr_grid_golden.npz"))
        shapes = [tuple(int(v) for v in s) for s in G2["shapes"]]
        F, P, bs = G2[f"F_{T}"], G2[f"P_{T}"], BS[T]
        enc, o = [], 0
        for k, (nr, npr) in enumerate(shapes):
            n = nr * npr // 256 * bs
            enc.append((F[o:o + n], P[o:o + n], int(G2["seed_offs"][k]), 30, npr, int(G2["imx_offs"][k]))); o += n
        seed, imx, want = G2["seed_bits"].view(np.uint8), G2["imx"], G2[f"B_{T}_2"].tobytes()
    else:
        enc, _ = _items(T)
        seed, imx, want = G["seed_bits"].view(np.uint8), None, G[f"B_{T}_2"].tobytes()
    nseg = len(_layout(T, [len(it[0]) // BS[T] for it in enc])[1])
    assert nseg >= 2
    for world in (2, 3):
        parts = [c.hist(T, enc, seed, imx, MODEL, shard.segment_range(nseg, r, world)) for r in range(world)]
        freq, used = normalize(sum(p[1] for p in parts))
        coded = [c.code(p[0], freq, used) for p in parts]
        got = c.finish(freq, used, np.concatenate([x[0] for x in coded]), b"".join(x[1] for x in coded), MODEL)
        assert got == want, f"world {world}"
