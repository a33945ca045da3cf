"""zstd over the system libzstd (ctypes), with the part of the `zstandard` Python package's interface that the
reference's host code uses (requirements.txt pins zstandard==0.25.0; that package is not available everywhere,
the C library is).  The module can be registered under the name `zstandard` so that the reference's container,
framing and repository code run on it unchanged:

    one-shot            compress(data, level) / decompress(data, max_output_size)     codecs_gguf.py:72-83
    ZstdCompressor      level= | compression_params=, dict_data=; .compress(), .compressobj(size=)
                                                                                      repo3.py:1518, 1536-1544, 1946-1948
    ZstdCompressionParameters.from_level(level, window_log=, enable_ldm=, threads=)   repo3.py:1513, 1533-1534, 1596-1597
    ZstdCompressionDict(data, dict_type=DICT_TYPE_RAWCONTENT)                         repo3.py:615, 2330
    ZstdDecompressor    dict_data=; .decompress(), .stream_reader(src, read_size=).readinto()
                                                                                      repo3.py:50-67, 330-364, container.py:146

A raw-content dictionary is given to libzstd as a prefix of the frame (ZSTD_CCtx_refPrefix / ZSTD_DCtx_refPrefix),
which is what a raw-content dictionary is.  Buffers go to the library by address (no copies in); every call
releases the GIL, so compression runs beside the GPU work as in the reference's pipelines.
"""
import ctypes
import ctypes.util
import os

import numpy as np

_lib = None

# ZSTD_cParameter / ZSTD_dParameter / ZSTD_EndDirective values of zstd.h (stable API)
_C_LEVEL, _C_WINDOWLOG, _C_LDM, _C_CONTENTSIZE, _C_NBWORKERS = 100, 101, 160, 200, 400
_D_WINDOWLOGMAX = 100
_E_CONTINUE, _E_FLUSH, _E_END = 0, 1, 2
_UNKNOWN, _ERROR = 0xffffffffffffffff, 0xfffffffffffffffe


class _Buf(ctypes.Structure):             # ZSTD_inBuffer and ZSTD_outBuffer share this layout
    _fields_ = [("ptr", ctypes.c_void_p), ("size", ctypes.c_size_t), ("pos", ctypes.c_size_t)]


def _z():
    global _lib
    if _lib is None:
        name = ctypes.util.find_library("zstd") or "libzstd.so.1"
        L = ctypes.CDLL(name)
        Z, P, I, U = ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
        sig = {
            "ZSTD_compressBound": (Z, [Z]), "ZSTD_isError": (ctypes.c_uint, [Z]), "ZSTD_getErrorName": (ctypes.c_char_p, [Z]),
            "ZSTD_getFrameContentSize": (U, [P, Z]),
            "ZSTD_createCCtx": (P, []), "ZSTD_freeCCtx": (Z, [P]), "ZSTD_CCtx_setParameter": (Z, [P, I, I]),
            "ZSTD_CCtx_setPledgedSrcSize": (Z, [P, U]), "ZSTD_CCtx_refPrefix": (Z, [P, P, Z]),
            "ZSTD_compress2": (Z, [P, P, Z, P, Z]), "ZSTD_compressStream2": (Z, [P, ctypes.POINTER(_Buf), ctypes.POINTER(_Buf), I]),
            "ZSTD_CStreamOutSize": (Z, []),
            "ZSTD_createDCtx": (P, []), "ZSTD_freeDCtx": (Z, [P]), "ZSTD_DCtx_setParameter": (Z, [P, I, I]),
            "ZSTD_DCtx_refPrefix": (Z, [P, P, Z]), "ZSTD_decompressDCtx": (Z, [P, P, Z, P, Z]),
            "ZSTD_decompressStream": (Z, [P, ctypes.POINTER(_Buf), ctypes.POINTER(_Buf)]),
        }
        for n, (res, args) in sig.items():
            f = getattr(L, n)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


class ZstdError(Exception):
    pass


def _ok(code):
    L = _z()
    if L.ZSTD_isError(code):
        raise ZstdError(L.ZSTD_getErrorName(code).decode())
    return code


def _view(data):
    """any bytes-like object as a uint8 array (no copy; read-only sources included)"""
    if isinstance(data, np.ndarray):
        return np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    return np.frombuffer(data, np.uint8)


def _addr(a):
    return ctypes.c_void_p(a.ctypes.data if a.size else 0)


# ---- parameters, dictionaries ---------------------------------------------------------------------------------------
DICT_TYPE_AUTO, DICT_TYPE_RAWCONTENT, DICT_TYPE_FULLDICT = 0, 1, 2


class ZstdCompressionParameters:
    def __init__(self, level=3, window_log=0, enable_ldm=False, threads=0):
        self.level, self.window_log, self.enable_ldm = level, window_log, bool(enable_ldm)
        self.threads = (os.cpu_count() or 1) if threads < 0 else threads

    @classmethod
    def from_level(cls, level, window_log=0, enable_ldm=False, threads=0, **kw):
        if kw:
            raise NotImplementedError(f"zstd parameters {sorted(kw)} are not part of this binding")
        return cls(level, window_log, enable_ldm, threads)


class ZstdCompressionDict:
    def __init__(self, data, dict_type=DICT_TYPE_AUTO):
        if dict_type != DICT_TYPE_RAWCONTENT:
            raise NotImplementedError("only raw-content dictionaries are part of this binding")
        self.data = bytes(data)
        self._arr = np.frombuffer(self.data, np.uint8)

    def as_bytes(self):
        return self.data


class _CCtx:
    """a compression context with parameters (and prefix) applied; freed with the object"""

    def __init__(self, params, dict_data, size=None):
        L = _z()
        self.L, self.c = L, L.ZSTD_createCCtx()
        if not self.c:
            raise MemoryError("ZSTD_createCCtx")
        self.keep = dict_data
        _ok(L.ZSTD_CCtx_setParameter(self.c, _C_LEVEL, params.level))
        if params.window_log:
            _ok(L.ZSTD_CCtx_setParameter(self.c, _C_WINDOWLOG, params.window_log))
        if params.enable_ldm:
            _ok(L.ZSTD_CCtx_setParameter(self.c, _C_LDM, 1))
        if params.threads:
            # the frame does not depend on the number of workers (the jobs' size follows from the window), only
            # on whether the multi-threaded coder is used at all
            _ok(L.ZSTD_CCtx_setParameter(self.c, _C_NBWORKERS, params.threads))
        _ok(L.ZSTD_CCtx_setParameter(self.c, _C_CONTENTSIZE, 1))
        if size is not None:
            _ok(L.ZSTD_CCtx_setPledgedSrcSize(self.c, size))
        if dict_data is not None:
            _ok(L.ZSTD_CCtx_refPrefix(self.c, _addr(dict_data._arr), dict_data._arr.size))

    def __del__(self):
        if getattr(self, "c", None):
            self.L.ZSTD_freeCCtx(self.c)
            self.c = None


class ZstdCompressor:
    def __init__(self, level=3, compression_params=None, dict_data=None, **kw):
        self.params = compression_params if compression_params is not None else ZstdCompressionParameters(level)
        self.dict_data = dict_data

    def compress(self, data):
        src = _view(data)
        cx = _CCtx(self.params, self.dict_data)
        cap = cx.L.ZSTD_compressBound(src.size)
        out = np.empty(cap, np.uint8)
        n = _ok(cx.L.ZSTD_compress2(cx.c, _addr(out), cap, _addr(src), src.size))
        return out[:n].tobytes()

    def compressobj(self, size=-1):
        return _CompressObj(_CCtx(self.params, self.dict_data, None if size is None or size < 0 else size))


class _CompressObj:
    def __init__(self, cx):
        self.cx = cx
        self.out = np.empty(max(cx.L.ZSTD_CStreamOutSize(), 1 << 20), np.uint8)

    def _run(self, src, mode):
        L, parts = self.cx.L, []
        ib = _Buf(src.ctypes.data if src.size else 0, src.size, 0)
        while True:
            ob = _Buf(self.out.ctypes.data, self.out.size, 0)
            left = _ok(L.ZSTD_compressStream2(self.cx.c, ctypes.byref(ob), ctypes.byref(ib), mode))
            if ob.pos:
                parts.append(self.out[:ob.pos].tobytes())
            if mode == _E_CONTINUE:
                if ib.pos == ib.size:
                    break
            elif left == 0:
                break
        return b"".join(parts)

    def compress(self, data):
        return self._run(_view(data), _E_CONTINUE)

    def flush(self):
        return self._run(np.empty(0, np.uint8), _E_END)


class _DCtx:
    def __init__(self, dict_data):
        L = _z()
        self.L, self.d = L, L.ZSTD_createDCtx()
        if not self.d:
            raise MemoryError("ZSTD_createDCtx")
        self.keep = dict_data
        _ok(L.ZSTD_DCtx_setParameter(self.d, _D_WINDOWLOGMAX, 31))
        if dict_data is not None:
            _ok(L.ZSTD_DCtx_refPrefix(self.d, _addr(dict_data._arr), dict_data._arr.size))

    def __del__(self):
        if getattr(self, "d", None):
            self.L.ZSTD_freeDCtx(self.d)
            self.d = None


class ZstdDecompressor:
    def __init__(self, dict_data=None, **kw):
        self.dict_data = dict_data

    def decompress(self, data, max_output_size=0):
        src = _view(data)
        L = _z()
        size = L.ZSTD_getFrameContentSize(_addr(src), src.size)
        if size == _ERROR:
            raise ZstdError("not a zstd frame")
        dx = _DCtx(self.dict_data)
        if size != _UNKNOWN:
            out = np.empty(max(1, size), np.uint8)
            n = _ok(L.ZSTD_decompressDCtx(dx.d, _addr(out), size, _addr(src), src.size))
            return out[:n].tobytes()
        if not max_output_size:
            raise ZstdError("frame does not record its size")
        r = _StreamReader(dx, src, 1 << 20)          # size not recorded: decoded piece by piece
        parts, total = [], 0
        while True:
            buf = bytearray(1 << 22)
            k = r.readinto(buf)
            if not k:
                break
            total += k
            if total > max_output_size:
                raise ZstdError("frame decodes to more than max_output_size")
            parts.append(bytes(buf[:k]))
        return b"".join(parts)

    def stream_reader(self, source, read_size=1 << 17, **kw):
        return _StreamReader(_DCtx(self.dict_data), source, read_size)


class _StreamReader:
    """forward reader of one frame: readinto(buf) fills buf as far as the frame goes"""

    def __init__(self, dx, source, read_size):
        self.dx, self.read_size = dx, read_size
        self.src = None if hasattr(source, "read") or hasattr(source, "readinto") else _view(source)
        self.f = source if self.src is None else None
        self.chunk, self.ib = np.empty(0, np.uint8), _Buf(0, 0, 0)
        self.spos, self.done = 0, False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def close(self):
        self.dx = None

    def _more(self):
        """next piece of the compressed input -> False at its end"""
        if self.src is not None:
            if self.spos >= self.src.size:
                return False
            self.chunk = self.src[self.spos:self.spos + self.read_size]
            self.spos += self.chunk.size
        else:
            if hasattr(self.f, "readinto"):
                buf = np.empty(self.read_size, np.uint8)
                k = self.f.readinto(memoryview(buf))
                self.chunk = buf[:k or 0]
            else:
                self.chunk = np.frombuffer(self.f.read(self.read_size), np.uint8)
            if not self.chunk.size:
                return False
        self.ib = _Buf(self.chunk.ctypes.data, self.chunk.size, 0)
        return True

    def readinto(self, b):
        out = np.frombuffer(b, np.uint8)
        if self.done or not out.size:
            return 0
        L = self.dx.L
        ob = _Buf(out.ctypes.data, out.size, 0)
        while ob.pos < ob.size:
            fed = self.ib.pos < self.ib.size or self._more()
            before = ob.pos
            r = _ok(L.ZSTD_decompressStream(self.dx.d, ctypes.byref(ob), ctypes.byref(self.ib)))
            if r == 0:                          # the frame is complete
                self.done = True
                break
            if not fed and ob.pos == before:    # input at its end and nothing left inside the decoder
                break
        return ob.pos

    def read(self, n=-1):
        if n is None or n < 0:
            parts = []
            while True:
                buf = bytearray(1 << 22)
                k = self.readinto(buf)
                if not k:
                    return b"".join(parts)
                parts.append(bytes(buf[:k]))
        buf = bytearray(n)
        return bytes(buf[:self.readinto(buf)])


# ---- one-shot helpers ---------------------------------------------------------------------------------------------
def compress(data, level=3):
    return ZstdCompressor(level=level).compress(data)


def decompress(data, max_output_size=0):
    return ZstdDecompressor().decompress(data, max_output_size)
