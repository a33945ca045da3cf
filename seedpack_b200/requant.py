"""Type table of the quantisers (host side).

`QFUN` keeps the name and meaning of seedpack/requant.py:21-27.  The importance-matrix loaders of that file
(:59-112) are host code that stays the reference's; its CPU quantiser binding (:114-134) has no counterpart
here - quantisation runs on the GPU only (see gpuquant.GPUQuant).
"""

# ggml type -> (function name, block elements, block bytes)
QFUN = {2: ("quantize_q4_0", 32, 18), 3: ("quantize_q4_1", 32, 20), 6: ("quantize_q5_0", 32, 22),
        7: ("quantize_q5_1", 32, 24), 8: ("quantize_q8_0", 32, 34), 10: ("quantize_q2_K", 256, 84),
        11: ("quantize_q3_K", 256, 110), 12: ("quantize_q4_K", 256, 144), 13: ("quantize_q5_K", 256, 176),
        14: ("quantize_q6_K", 256, 210), 16: ("quantize_iq2_xxs", 256, 66), 17: ("quantize_iq2_xs", 256, 74),
        18: ("quantize_iq3_xxs", 256, 98), 19: ("quantize_iq1_s", 256, 50), 20: ("quantize_iq4_nl", 32, 18),
        21: ("quantize_iq3_s", 256, 110), 22: ("quantize_iq2_s", 256, 82), 23: ("quantize_iq4_xs", 256, 136),
        29: ("quantize_iq1_m", 256, 56), 42: ("quantize_q2_0", 64, 18),
        # beyond the reference's own table: the remaining quantize_* of ggml-quants.c (no importance matrix, no dequantiser here)
        34: ("quantize_tq1_0", 256, 54), 35: ("quantize_tq2_0", 256, 66), 39: ("quantize_mxfp4", 32, 17),
        40: ("quantize_nvfp4", 64, 36), 41: ("quantize_q1_0", 128, 18)}
# types whose quantiser refuses to run without an importance matrix
NEEDS_IMATRIX = {16, 17, 19}
# (type, variant) pairs beyond variant 0 (seedpack/gpuquant.py:182-185)
VARIANTS = {29: 1}
