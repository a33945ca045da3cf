"""CPU checks of the checkers: the plain-C restatement (oracle/quants_port.c) and the compiled reference C code
(oracle/_ref) against the golden vectors produced by the reference's own --cpu path
(tests/golden/quant_golden.npz, written by tests/golden/make_quant_golden.py), and against each other."""
import os

import numpy as np
import pytest

from oracle import port, ref
from tests import synth

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = np.load(os.path.join(HERE, "golden", "quant_golden.npz"))
BITS, IMX = GOLD["bits"], GOLD["imatrix"]
X = synth.bf16_bits_to_f32(BITS).reshape(BITS.shape)
KEYS = [k for k in GOLD.files if k.startswith("t")]


def _case(key):
    t, use, v = key[1:].split("_")
    return int(t), use == "imx", int(v[1:])


@pytest.mark.parametrize("key", [k for k in KEYS if _case(k)[0] in port.PORT_TYPES])
def test_port_matches_golden(key):
    t, use, _ = _case(key)
    assert np.array_equal(port.quantize(t, X, IMX if use else None), GOLD[key])


@pytest.mark.parametrize("key", KEYS)
def test_compiled_reference_matches_golden(key):
    if not ref.available():
        pytest.skip("oracle/_ref not built (needs the reference tree)")
    t, use, v = _case(key)
    assert np.array_equal(ref.quantize(t, X, IMX if use else None, variant=v), GOLD[key])


def test_fp16_conversion_exhaustive_f16_side():
    """all 65536 half patterns: to float and back is the identity (NaNs map to the canonical 0x7e00 | sign)"""
    L = port.lib()
    for h in range(0, 65536, 1):
        f = L.op_f16_to_f32(h)
        back = L.op_f32_to_f16(f)
        if (h & 0x7c00) == 0x7c00 and (h & 0x3ff):
            assert back == ((h & 0x8000) | 0x7e00)
        else:
            assert back == h


def test_fp16_conversion_matches_numpy_rounding():
    """round-to-nearest-even on a dense sample, checked against numpy's float16 cast"""
    L = port.lib()
    rng = np.random.default_rng(3)
    v = np.concatenate([rng.normal(0, 1, 20000), rng.normal(0, 1e-4, 20000), rng.normal(0, 1e-7, 20000),
                        rng.normal(0, 3e4, 20000), [0.0, -0.0, 65504.0, 65520.0, 1e-8, 6.0e-8]]).astype(np.float32)
    want = v.astype(np.float16).view(np.uint16)
    got = np.array([L.op_f32_to_f16(float(a)) for a in v], np.uint16)
    assert np.array_equal(got, want)


def test_nearest_int_matches_round_half_even():
    L = port.lib()
    rng = np.random.default_rng(4)
    v = np.concatenate([rng.uniform(-4e6, 4e6, 50000), np.arange(-100, 100) + 0.5, rng.normal(0, 3, 50000)]).astype(np.float32)
    want = np.rint(v.astype(np.float64)).astype(np.int64)
    got = np.array([L.op_nearest_int(float(a)) for a in v], np.int64)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("t", sorted(port.PORT_TYPES))
def test_port_matches_compiled_reference_on_edge_rows(t):
    if not ref.available():
        pytest.skip("oracle/_ref not built (needs the reference tree)")
    bits = synth.weights(16, 1024, seed=500 + t)
    x = synth.bf16_bits_to_f32(bits).reshape(16, 1024)
    imx = synth.imatrix(1024, seed=t)
    for w in (imx, None):
        assert np.array_equal(port.quantize(t, x, w), ref.quantize(t, x, w))
