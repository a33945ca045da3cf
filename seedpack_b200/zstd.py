"""Minimal zstd binding over the system libzstd (ctypes): the `zstandard` Python package the reference uses
(requirements.txt: zstandard==0.25.0) is not available everywhere, the C library is.  Only what the coded-batch
framing needs: one-shot compress at a level and one-shot decompress (seedpack/codecs_gguf.py:72-83).

The module also exposes the handful of names of the `zstandard` API that the reference's modules touch at import
or in those two calls, so that test tooling can register it under that name to import the reference."""
import ctypes
import ctypes.util

_lib = None


def _z():
    global _lib
    if _lib is None:
        name = ctypes.util.find_library("zstd") or "libzstd.so.1"
        L = ctypes.CDLL(name)
        L.ZSTD_compressBound.restype = ctypes.c_size_t
        L.ZSTD_compressBound.argtypes = [ctypes.c_size_t]
        L.ZSTD_compress.restype = ctypes.c_size_t
        L.ZSTD_compress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int]
        L.ZSTD_decompress.restype = ctypes.c_size_t
        L.ZSTD_decompress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t]
        L.ZSTD_getFrameContentSize.restype = ctypes.c_ulonglong
        L.ZSTD_getFrameContentSize.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        L.ZSTD_isError.restype = ctypes.c_uint
        L.ZSTD_isError.argtypes = [ctypes.c_size_t]
        L.ZSTD_getErrorName.restype = ctypes.c_char_p
        L.ZSTD_getErrorName.argtypes = [ctypes.c_size_t]
        _lib = L
    return _lib


class ZstdError(Exception):
    pass


def compress(data, level=3):
    L = _z()
    data = bytes(data)
    cap = L.ZSTD_compressBound(len(data))
    buf = ctypes.create_string_buffer(cap)
    n = L.ZSTD_compress(buf, cap, data, len(data), level)
    if L.ZSTD_isError(n):
        raise ZstdError(L.ZSTD_getErrorName(n).decode())
    return buf.raw[:n]


def decompress(data, max_output_size=0):
    L = _z()
    data = bytes(data)
    size = L.ZSTD_getFrameContentSize(data, len(data))
    if size in (0xffffffffffffffff, 0xfffffffffffffffe):        # unknown / error
        if not max_output_size:
            raise ZstdError("frame does not record its size")
        size = max_output_size
    buf = ctypes.create_string_buffer(max(1, size))
    n = L.ZSTD_decompress(buf, size, data, len(data))
    if L.ZSTD_isError(n):
        raise ZstdError(L.ZSTD_getErrorName(n).decode())
    return buf.raw[:n]


# ---- the subset of the `zstandard` package API used by one-shot callers -------------------------------------
DICT_TYPE_RAWCONTENT = 1


class ZstdCompressionParameters:
    def __init__(self, level):
        self.level = level

    @classmethod
    def from_level(cls, level, **kw):
        return cls(level)


class ZstdCompressionDict:
    def __init__(self, data, dict_type=None):
        self.data = bytes(data)


class ZstdCompressor:
    def __init__(self, level=3, compression_params=None, dict_data=None, **kw):
        if dict_data is not None:
            raise NotImplementedError("dictionary compression is not part of this binding")
        self.level = compression_params.level if compression_params is not None else level

    def compress(self, data):
        return compress(data, self.level)


class ZstdDecompressor:
    def __init__(self, dict_data=None, **kw):
        if dict_data is not None:
            raise NotImplementedError("dictionary decompression is not part of this binding")

    def decompress(self, data, max_output_size=0):
        return decompress(data, max_output_size)
