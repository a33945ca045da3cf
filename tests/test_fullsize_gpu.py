"""Properties that do not depend on the size, checked at the benchmark's full size (one BF16 tensor of 4096 x 12288 with
its importance matrix, seeded): the CPU checker would need minutes per type there, so these tests lean on what must
hold whatever the size - rows are independent, a coded batch decodes to what was coded, coding does not depend on how
the work was cut."""
import numpy as np
import pytest

from tests import synth

pytestmark = pytest.mark.gpu
NROWS, NPR = 4096, 12288


@pytest.fixture(scope="module")
def tensor():
    import torch
    bits = synth.weights(NROWS, NPR, 1, edge_cases=False)
    imx = synth.imatrix(NPR, 1)
    x = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16).reshape(-1)
    return bits, imx, x


# the benchmark's 40 launches: every type of the reference's table with the importance matrix, the 15 whose matrix-free
# routine is another code path, and the 5 further quantisers, which take none
_ALL = [2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 16, 17, 18, 19, 20, 21, 22, 23, 29, 42]
CASES = [(t, True) for t in _ALL] + [(t, False) for t in (2, 3, 6, 7, 10, 11, 12, 13, 14, 18, 20, 21, 22, 23, 29, 34, 35, 39, 40, 41)]


@pytest.mark.parametrize("t,use", CASES)
def test_rows_are_independent_at_full_size(tensor, t, use):
    """the whole tensor in one launch gives the bytes of its two halves quantised on their own, and five of its rows
    (12288 weights each: 48 super-blocks, the whole-row mean square of the legacy importance paths) equal the
    reference's C code"""
    import torch
    from oracle import ref
    from seedpack_b200.gpuquant import GPUQuant
    from seedpack_b200.requant import QFUN
    bits, imx, x = tensor
    gq = GPUQuant()
    w = imx if use else None
    whole = gq.quantize_tensors(t, [(x, NPR)], [w], device=True)[0]
    half = NROWS // 2 * NPR
    a, b = gq.quantize_tensors(t, [(x[:half], NPR), (x[half:], NPR)], [w, w], device=True)
    assert torch.equal(whole, torch.cat([a, b]))
    assert gq.status() == 0
    if ref.available():
        _, qk, bs = QFUN[t]
        rb = NPR // qk * bs
        rows = (0, 1, 2047, 2048, 4095)
        h = torch.cat([whole[r * rb:(r + 1) * rb] for r in rows]).cpu().numpy()
        for k, r in enumerate(rows):
            want = ref.quantize(t, synth.bf16_bits_to_f32(bits[r:r + 1]).reshape(1, NPR), w, threads=1)
            assert np.array_equal(h[k * rb:(k + 1) * rb], want), (t, use, r)


@pytest.mark.parametrize("T", [12, 17])
def test_qr_round_trip_at_full_size(tensor, T):
    """a coded batch of the full tensor decodes to the file, and the single-pass and the staged encoder agree"""
    from seedpack_b200.gpuquant import GPUQuant
    from seedpack_b200.qr import GRID_TYPES, QRCodec
    bits, imx, x = tensor
    gq = GPUQuant()
    rng = np.random.default_rng(5)
    imx2 = (imx * np.exp(rng.normal(0, 0.3, imx.shape))).astype(np.float32)
    P = gq.quantize_tensors(T, [(x, NPR)], [imx])[0]
    F = gq.quantize_tensors(T, [(x, NPR)], [imx2])[0].copy()
    F[::997] ^= 0x5a
    seed = bits.view(np.uint8).reshape(-1)
    gim = imx if T in GRID_TYPES else None
    ioff = 0 if T in GRID_TYPES else -1
    buf = QRCodec().encode(T, [(F, P, 0, 30, NPR, ioff)], seed, gim)
    out = QRCodec().decode(T, buf, [(P, 0, 30, NPR, ioff)], seed, gim)
    assert np.array_equal(out.cpu().numpy(), F)
    if T == 12:
        assert QRCodec(staged=False).encode(T, [(F, P, 0, 30, NPR, ioff)], seed, gim) == buf


def test_r2_round_trip_and_grouping_at_full_size(tensor):
    """the R2 coding of a file holding the full tensor (as two tensors of one role) decodes to its bytes, and does not
    depend on the group size; the reference's BF16v2 class over the bound kernels"""
    from seedpack_b200 import refbind, synthrepo
    if not refbind.available():
        pytest.fail("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE)")
    refbind.install()
    from seedpack import bf16v2, codecs_gguf
    bits, _, _ = tensor
    half = NROWS // 2
    data = synthrepo.gguf_bytes([("general.alignment", 4, 32)],
                                [(f"blk.{k}.ffn_up.weight", (NPR, half), 30, half * NPR * 2, (lambda k=k: bits[k * half:(k + 1) * half])) for k in range(2)])
    parts = codecs_gguf.unpack(b"".join(bytes(p) for p in bf16v2.BF16v2().compress_parts(data)))
    small = codecs_gguf.unpack(b"".join(bytes(p) for p in bf16v2.BF16v2(group_bytes=half * NPR * 2).compress_parts(data)))
    for k in ("stream", "tables", "side"):
        assert bytes(parts[k]) == bytes(small[k]), k
    back = bf16v2.BF16v2().decompress(codecs_gguf.pack({k: bytes(v) for k, v in parts.items()}))
    assert np.array_equal(np.asarray(back), np.frombuffer(data, np.uint8))


def test_rans_round_trip_on_a_large_stream():
    import torch
    from seedpack_b200.rans import RansCodec
    n, ntab = 1 << 27, 294
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    sym = torch.where(torch.rand(n, generator=g, device="cuda") < 0.97, 0, torch.randint(0, 64, (n,), generator=g, device="cuda")).to(torch.uint8)
    tab = torch.randint(0, 292, (n // 32,), generator=g, device="cuda").to(torch.int16)
    c = RansCodec()
    r = c.encode(sym, tab, 32, ntab)
    out = c.decode(r["stream"], r["off"], tab, 32, n, r["freq"], r["used"], ntab)
    assert torch.equal(out, sym) and c.status() == 0
