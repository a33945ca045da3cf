"""GPU parity: every re-quantiser against the reference's own C code (oracle/_ref), byte for byte,
through the C ABI (seedpack_b200.gpuquant -> libseedgrow.so)."""
import numpy as np
import pytest

from oracle import ref
from tests import synth

pytestmark = pytest.mark.gpu

TYPES = sorted(ref.QFUN)
CASES = [(t, imx) for t in TYPES for imx in ((True,) if t in ref.NEEDS_IMATRIX else (True, False))]


@pytest.fixture(scope="module")
def gq():
    from seedpack_b200.gpuquant import GPUQuant
    return GPUQuant()


def _diff_report(t, a, b):
    name, qk, bs = ref.QFUN[t]
    bad = np.flatnonzero(a != b)
    blocks = np.unique(bad // bs)
    first = int(blocks[0])
    return (f"{name}: {bad.size} bytes differ in {blocks.size} of {a.size // bs} blocks; first block {first}: "
            f"byte offsets {sorted(set((bad[bad // bs == first] % bs).tolist()))[:16]}\n"
            f"  gpu {a[first * bs:(first + 1) * bs].tolist()}\n  ref {b[first * bs:(first + 1) * bs].tolist()}")


@pytest.mark.parametrize("t,with_imx", CASES)
def test_quantize_matches_reference(gq, t, with_imx):
    import torch
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    nrows, npr = 24, 1024
    bits = synth.weights(nrows, npr, seed=100 + t)
    imx = synth.imatrix(npr, seed=t) if with_imx else None
    want = ref.quantize(t, synth.bf16_bits_to_f32(bits).reshape(nrows, npr), imx)
    x = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    got = gq.quantize_tensors(t, [(x.reshape(-1), npr)], [imx])[0]
    assert gq.status() == 0
    assert got.size == want.size
    assert np.array_equal(got, want), _diff_report(t, np.asarray(got), want)


@pytest.mark.parametrize("t", [8, 2, 12, 14])
def test_source_dtypes_agree(gq, t):
    """bf16, f16 and f32 sources holding the same values give the same bytes"""
    import torch
    nrows, npr = 8, 512
    bits = synth.weights(nrows, npr, seed=5, edge_cases=False)
    xb = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16).reshape(-1)
    x32 = xb.float()
    x16 = x32.half()                         # lossy, so compare f16 against f32 of the same f16 values
    a = gq.quantize_tensors(t, [(xb, npr)], [None])[0]
    b = gq.quantize_tensors(t, [(x32, npr)], [None])[0]
    c = gq.quantize_tensors(t, [(x16, npr)], [None])[0]
    d = gq.quantize_tensors(t, [(x16.float(), npr)], [None])[0]
    assert np.array_equal(a, b)
    assert np.array_equal(c, d)


def test_ragged_multi_tensor_launch(gq):
    """several tensors of different shapes in one call, legacy rows that are not multiples of 256"""
    import torch
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    shapes = [(3, 96), (5, 1024), (1, 32), (7, 288), (2, 2048)] * 4          # 20 tensors: more than one launch group
    for t in (2, 3, 8, 6):
        srcs, imxs, wants = [], [], []
        for k, (nr, npr) in enumerate(shapes):
            bits = synth.weights(nr, npr, seed=k, edge_cases=False)
            imx = synth.imatrix(npr, seed=k) if k % 2 == 0 else None
            srcs.append((torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16).reshape(-1), npr))
            imxs.append(imx)
            wants.append(ref.quantize(t, synth.bf16_bits_to_f32(bits).reshape(nr, npr), imx))
        got = gq.quantize_tensors(t, srcs, imxs)
        for g, w in zip(got, wants):
            assert np.array_equal(g, w)


@pytest.mark.parametrize("with_imx", [True, False])
def test_iq1_m_variant_1(gq, with_imx):
    """the older IQ1_M split search (direct sums instead of prefix sums) is a separate variant"""
    import torch
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    nrows, npr = 16, 1024
    bits = synth.weights(nrows, npr, seed=77)
    imx = synth.imatrix(npr, seed=3) if with_imx else None
    x32 = synth.bf16_bits_to_f32(bits).reshape(nrows, npr)
    want = ref.quantize(29, x32, imx, variant=1)
    x = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    got = gq.quantize_tensors(29, [(x.reshape(-1), npr)], [imx], variant=1)[0]
    assert gq.status() == 0
    assert np.array_equal(got, want), _diff_report(29, np.asarray(got), want)


def test_quantize_matches_golden_vectors(gq):
    """outputs of the reference's own --cpu path, committed under tests/golden/"""
    import os
    import torch
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_golden.npz"))
    bits, imx = gold["bits"], gold["imatrix"]
    x = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16).reshape(-1)
    for key in gold.files:
        if not key.startswith("t"):
            continue
        t, use, v = key[1:].split("_")
        got = gq.quantize_tensors(int(t), [(x, bits.shape[1])], [imx if use == "imx" else None], variant=int(v[1:]))[0]
        assert np.array_equal(got, gold[key]), key
    assert gq.status() == 0


@pytest.mark.parametrize("t", TYPES)
def test_dequantize_matches_reference(gq, t):
    """dequantised floats equal the reference's dequantize_row_<type> bit for bit (blocks = quantiser output)"""
    import torch
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    nrows, npr = 12, 1024
    bits = synth.weights(nrows, npr, seed=40 + t)
    imx = synth.imatrix(npr, seed=t)
    y = ref.quantize(t, synth.bf16_bits_to_f32(bits).reshape(nrows, npr), imx)
    want = ref.dequantize(t, y, nrows * npr)
    got = gq.dequantize(t, torch.from_numpy(y).cuda()).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_convert_float(gq):
    import torch
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.normal(0, 1, 5000), rng.normal(0, 1e-6, 1000), [0.0, -0.0, 65504.0, 1e-8, 3.0e38]]).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    b = gq.convert_float(xd, torch.bfloat16)
    assert np.array_equal(b.view(torch.int16).cpu().numpy().view(np.uint16), synth.f32_to_bf16_bits(x))
    h = gq.convert_float(xd, torch.float16)
    with np.errstate(over="ignore"):
        assert np.array_equal(h.view(torch.int16).cpu().numpy().view(np.uint16), x.astype(np.float16).view(np.uint16))
    back = gq.convert_float(b, torch.float32)
    assert np.array_equal(back.cpu().numpy(), synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(x)))


def test_extra_types_match_golden(gq):
    """TQ1_0, TQ2_0, MXFP4, NVFP4, Q1_0 against bytes and dequantised values the reference's C code produced
    (tests/golden/quant_extra_golden.npz)"""
    import os
    import torch
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_extra_golden.npz"))
    npr = int(g["npr"])
    x = torch.from_numpy(g["bits"].view(np.int16)).cuda().view(torch.bfloat16).reshape(-1)
    for t in (34, 35, 39, 40, 41):
        got = gq.quantize_tensors(t, [(x, npr)], [None])[0]
        assert np.array_equal(got, g[f"q_{t}"]), _diff_report(t, np.asarray(got), g[f"q_{t}"])
        back = gq.dequantize(t, torch.from_numpy(g[f"q_{t}"]).cuda()).cpu().numpy()
        assert np.array_equal(back.view(np.uint32), g[f"d_{t}"].view(np.uint32)), t
        # float32 sources holding the same values give the same bytes
        assert np.array_equal(gq.quantize_tensors(t, [(x.float(), npr)], [None])[0], g[f"q_{t}"])
    assert gq.status() == 0
