"""Seeded synthetic inputs with the value laws of the benchmark configurations: weights N(0, 0.02^2) with
0.1 % outliers at +-20 sigma, rounded to bf16 with round-to-nearest-even on the bit pattern
(the integer formula of seedpack/repo3.py:687-688); importance matrices exp(N(0, 1.5^2))."""
import numpy as np


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7fff) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def weights(nrows, npr, seed, edge_cases=True):
    """(nrows, npr) uint16 bf16 bit patterns"""
    rng = np.random.default_rng(seed)
    x = rng.normal(0.0, 0.02, (nrows, npr)).astype(np.float32)
    m = rng.random((nrows, npr)) < 0.001
    x[m] = np.where(rng.random(int(m.sum())) < 0.5, np.float32(-0.4), np.float32(0.4))
    if edge_cases and nrows >= 8 and npr >= 512:
        x[1, :256] = 0.0                       # all-zero super-block
        x[2, 256:512] = x[2, 256]              # constant block: every comparison ties
        x[3, :32] = 0.0; x[3, 5] = 1e-3        # single non-zero weight
        x[4, 0] = 0.5                          # block maximum in the first position ...
        x[4, 287] = -0.5                       # ... and negative in the last position of a 32-block
        x[5, :64] = np.float32(1e-41)          # denormals
        x[6, :256] = np.abs(x[6, :256])        # all positive (min clamps to 0)
        x[7, :256] = -np.abs(x[7, :256])       # all negative
        x[0, 32:64] = np.where(np.arange(32) % 2 == 0, np.float32(0.0), np.float32(-0.0))   # signed zeros
    return f32_to_bf16_bits(x)


def imatrix(npr, seed):
    rng = np.random.default_rng(seed + 7919)
    return np.exp(rng.normal(0.0, 1.5, npr)).astype(np.float32)
