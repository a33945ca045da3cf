"""Device twins of host arrays.

The reference keeps a repository's files and its predictions in host arrays (its design for GPUs with a few GB of
memory) and moves bytes to the device whenever a kernel needs them.  Where the binding already has the same bytes on
the device - a prediction it has just downloaded, a span of a file it has uploaded to compare - it remembers the pair
here, by host address range, so that a later use of the host array (the block compare, the difference count, the QR
coder's inputs) runs on the device copy without another upload.  An entry lives as long as the host memory it mirrors
(a finalizer on the array that owns the memory) and at most until `CAP` bytes of twins are registered after it.

Only arrays that the reference does not write to after registration may be registered or looked up: predictions
(never written), and file spans between their upload and the coding of their tensors (seedpack/repo3.py:1071-1188
compares a QR tensor's region and hands it to the coder unchanged; it is zeroed only after qr.encode, repo3.py:534-537).
"""
import bisect
import threading
import weakref
from collections import OrderedDict

import numpy as np

CAP = 12 << 30
_lock = threading.RLock()          # re-entrant: a finalizer (_drop) may run inside register() when the collector wakes there
_starts = []                       # sorted start addresses
_ents = OrderedDict()              # start -> (end, device uint8 tensor), oldest first
_bytes = [0]


def _addr(a):
    return a.__array_interface__["data"][0]


def root(a):
    """the array that owns a's memory"""
    while isinstance(getattr(a, "base", None), np.ndarray):
        a = a.base
    return a


def _drop(s, dev):
    with _lock:
        e = _ents.get(s)
        if e is not None and e[1] is dev:
            del _ents[s]
            _bytes[0] -= e[0] - s
            i = bisect.bisect_left(_starts, s)
            if i < len(_starts) and _starts[i] == s:
                del _starts[i]


def register(host, dev):
    """host: a C-contiguous NumPy array; dev: uint8 CUDA tensor holding the same bytes"""
    s, n = _addr(host), host.nbytes
    if not n or dev.numel() != n:
        return
    with _lock:
        old = _ents.pop(s, None)
        if old is None:
            bisect.insort(_starts, s)
        else:
            _bytes[0] -= old[0] - s
        _ents[s] = (s + n, dev)
        _bytes[0] += n
        evict = []
        while _bytes[0] > CAP and len(_ents) > 1:
            s0, (e0, d0) = next(iter(_ents.items()))
            if s0 == s:
                break
            evict.append((s0, d0))
            if _ents.pop(s0, None) is None:
                continue
            _bytes[0] -= e0 - s0
            i = bisect.bisect_left(_starts, s0)
            if i < len(_starts) and _starts[i] == s0:
                del _starts[i]
    weakref.finalize(root(host), _drop, s, dev)


def find(a):
    """the device bytes of host array a (uint8 CUDA tensor), or None"""
    if not isinstance(a, np.ndarray) or not a.flags.c_contiguous or not a.nbytes:
        return None
    s, n = _addr(a), a.nbytes
    with _lock:
        i = bisect.bisect_right(_starts, s) - 1
        if i < 0:
            return None
        s0 = _starts[i]
        end, dev = _ents[s0]
        if s + n > end:
            return None
    return dev[s - s0:s - s0 + n]


def clear():
    with _lock:
        _starts.clear(); _ents.clear(); _bytes[0] = 0
