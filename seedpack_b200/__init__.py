"""seedpack_b200 - B200-native re-quantise / residual / rANS path behind a C ABI.

Host-side mirrors of the reference's operator interface live in `gpuquant` (quantisers) and
follow its names and argument meanings; all arithmetic runs in libseedgrow.so (CUDA, sm_100a).
"""
from ._lib import LIB_PATH, SgError, lib  # noqa: F401

__all__ = ["LIB_PATH", "SgError", "lib"]
