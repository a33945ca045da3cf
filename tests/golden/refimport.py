"""Test tooling: import the reference package (SEEDPACK_CPU=1, its kernels compiled for the host) in this
container.  The `zstandard` package it imports is absent; seedpack_b200.zstd (a ctypes binding of the system
libzstd) is registered under that name.  Only the golden-vector generators use this."""
import os
import sys


def setup(ref_tree):
    os.environ["SEEDPACK_CPU"] = "1"
    os.environ.setdefault("SEEDPACK_CACHE", "/tmp/seedpack-golden-cache")
    os.environ.setdefault("NUMBA_CACHE_DIR", "/tmp/seedpack-golden-numba")
    os.makedirs(os.environ["SEEDPACK_CACHE"], exist_ok=True)
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.normpath(os.path.join(here, "..", ".."))
    for p in (root, ref_tree):
        if p not in sys.path:
            sys.path.insert(0, p)
    from seedpack_b200 import zstd
    sys.modules.setdefault("zstandard", zstd)
