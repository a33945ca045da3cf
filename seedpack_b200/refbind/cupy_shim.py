"""The array / launch module the reference's host code sees in place of CuPy when its kernels are served by
libseedgrow.so (registered as `cupy` by seedpack_b200.refbind.install()).

The reference reaches the GPU through a narrow protocol (seedpack/xp.py:6-18): device arrays with CuPy's transfer
methods, `RawModule(code=...).get_function(name)(grid, block, args, shared_mem=)`, a memory-pool and a runtime
object.  Its own `--cpu` mode swaps in a NumPy stand-in for the same protocol (seedpack/cpu.py).  This module is a
third realisation of it:

  * `ndarray` - a C-contiguous array whose bytes live in device memory (a torch uint8 CUDA tensor), in host memory
    (a NumPy array), or both.  What moves tensor-sized data stays on the device: slices along the first axis,
    `view`, `reshape`, `get` / `set`, slice assignment, `concatenate`, row gathers / scatters.  Every other
    operation (the arithmetic on counts, tables, lengths and offsets: kilobytes) runs in NumPy on the host copy
    and gives a host-resident result that is uploaded when a kernel first needs it - the numbers are NumPy's, the
    same as the reference's `--cpu` mode computes, sorts stable as CuPy's are (seedpack/cpu.py:47-52).
  * `RawModule` - compiles nothing.  `get_function(name)` returns the binding of the reference's kernel `name` to
    the C ABI (seedpack_b200/refbind/kernels.py) or raises: no kernel source of the reference ever runs here.
  * `cuda`, memory pools, `cupyx.empty_pinned` - thin forwards to torch's caching allocators.

torch is the allocator and stream owner only; no torch operator computes anything that reaches the archive.
"""
import os
import threading
import types
import warnings
import weakref

import numpy as np
import torch

from . import xfer

_BIG = 1 << 16                     # arrays from this size on are created on the device
_SLACK = 64                        # device allocations are padded: vector loads may read up to the next 16 bytes
_DEBUG = os.environ.get("SEEDGROW_BIND_DEBUG") == "1"
STATS = {"d2h": 0, "h2d": 0, "host_ops": 0}
_LOCK = threading.RLock()          # residency changes of a storage (arrays are shared between the pipelines' threads)


# One process drives one GPU: the device that was current when the binding was installed.  torch's "current device" is
# a per-thread setting that starts at device 0 in every new thread, and the reference works from several threads
# (window preparation, the QR coder, the base coder): each of them is put on the bound device the first time it comes
# through here, so that no allocation or launch of a worker thread lands on another process's GPU.
DEVICE = None
_TLS = threading.local()


def bind_device(index=None):
    global DEVICE
    DEVICE = torch.cuda.current_device() if index is None else int(index)
    return DEVICE


def device_index():
    """the bound device's ordinal; the calling thread is switched to it"""
    if DEVICE is None:
        bind_device()
    if getattr(_TLS, "dev", None) != DEVICE:
        torch.cuda.set_device(DEVICE)
        _TLS.dev = DEVICE
    return DEVICE


def _device():
    return torch.device("cuda", device_index())


class _Storage:
    """the bytes behind one or more arrays: on the device, on the host, or on both"""
    __slots__ = ("n", "host", "dev", "hv", "dv", "zero", "__weakref__")

    def __init__(self, n, zero=False):
        self.n, self.host, self.dev, self.hv, self.dv, self.zero = int(n), None, None, False, False, zero

    def need_host(self):
        with _LOCK:
            return self._need_host()

    def need_dev(self):
        with _LOCK:
            return self._need_dev()

    def _need_host(self):
        if self.host is None:
            self.host = np.zeros(self.n, np.uint8) if (self.zero and not self.dv) else np.empty(self.n, np.uint8)
            if not self.dv:
                self.hv = True
        if not self.hv:
            if self.dv and self.n:
                xfer.d2h(self.host, self.dev[:self.n])
                STATS["d2h"] += self.n
            self.hv = True
        return self.host

    def _need_dev(self):
        if self.dev is None:
            cap = (self.n + _SLACK + 255) // 256 * 256
            if self.zero and not self.hv:
                self.dev = torch.zeros(cap, dtype=torch.uint8, device=_device())
            else:
                self.dev = torch.empty(cap, dtype=torch.uint8, device=_device())
            if not self.hv:
                self.dv = True
        if not self.dv:
            if self.hv and self.n:
                xfer.h2d(self.dev[:self.n], self.host)
                STATS["h2d"] += self.n
            self.dv = True
        return self.dev

    def wrote_host(self):
        self.hv, self.dv = True, False

    def wrote_dev(self):
        self.dv, self.hv = True, False

    @property
    def on_dev(self):
        return self.dv and not self.hv


class _Data:
    def __init__(self, a):
        self._a = a

    @property
    def ptr(self):
        return self._a.dev_in().data_ptr()


def _from_numpy(a):
    """torch view of a NumPy array that is only read (a read-only mapping of a file is fine)"""
    if a.flags.writeable:
        return torch.from_numpy(a)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return torch.from_numpy(a)


def _prod(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class ndarray:
    __slots__ = ("st", "off", "dtype", "shape", "__weakref__")
    __array_priority__ = 100
    __array_ufunc__ = None             # NumPy operands defer to this class's reflected operators

    def __init__(self, st, off, dtype, shape):
        self.st, self.off, self.dtype, self.shape = st, int(off), np.dtype(dtype), tuple(int(s) for s in shape)

    # ---- geometry ---------------------------------------------------------------------------------------
    @property
    def size(self):
        return _prod(self.shape)

    @property
    def itemsize(self):
        return self.dtype.itemsize

    @property
    def nbytes(self):
        return self.size * self.dtype.itemsize

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def data(self):
        return _Data(self)

    @property
    def T(self):
        return _wrap(self._h().T)

    def __len__(self):
        if not self.shape:
            raise TypeError("len() of a 0-d array")
        return self.shape[0]

    # ---- the two sides ---------------------------------------------------------------------------------
    def _h(self):
        """NumPy view of the host copy (made valid first)"""
        b = self.st.need_host()
        return b[self.off:self.off + self.nbytes].view(self.dtype).reshape(self.shape)

    def _hw(self):
        """NumPy view of the host copy for writing: the device copy is stale afterwards"""
        a = self._h()
        self.st.wrote_host()
        return a

    def dev_in(self):
        """torch uint8 view of the device copy (made valid first), for a kernel that reads it"""
        d = self.st.need_dev()
        return d[self.off:self.off + self.nbytes]

    def dev_out(self):
        """the same for a kernel that writes it: the host copy is stale afterwards.  An array that covers its whole
        storage is not uploaded first (every byte is about to be overwritten or is not read back)"""
        st = self.st
        with _LOCK:
            if self.nbytes == st.n and not st.zero:
                if st.dev is None:
                    st.dev = torch.empty((st.n + _SLACK + 255) // 256 * 256, dtype=torch.uint8, device=_device())
                st.dv, st.hv = True, False
                return st.dev[:st.n]
        d = self.dev_in()
        st.wrote_dev()
        return d

    def dev_inout(self):
        d = self.dev_in()
        self.st.wrote_dev()
        return d

    def _big_dev(self):
        return (self.st.dv and not self.st.hv) or (self.st.dev is None and self.st.host is None and self.st.n >= _BIG)

    # ---- views -------------------------------------------------------------------------------------------
    def view(self, dtype=None):
        dt = np.dtype(dtype)
        if dt.itemsize == self.dtype.itemsize:
            return ndarray(self.st, self.off, dt, self.shape)
        if not self.shape:
            raise ValueError("view of a 0-d array with another item size")
        last = self.shape[-1] * self.dtype.itemsize
        if last % dt.itemsize:
            raise ValueError("the last axis does not divide into the new item size")
        return ndarray(self.st, self.off, dt, self.shape[:-1] + (last // dt.itemsize,))

    def reshape(self, *shape, order="C"):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = [int(s) for s in shape]
        if -1 in shape:
            k = shape.index(-1)
            rest = _prod(s for i, s in enumerate(shape) if i != k)
            shape[k] = self.size // rest if rest else 0
        if _prod(shape) != self.size:
            raise ValueError(f"cannot reshape array of size {self.size} into shape {tuple(shape)}")
        return ndarray(self.st, self.off, self.dtype, shape)

    def ravel(self):
        return self.reshape(-1)

    flatten = ravel

    def _row_bytes(self):
        return _prod(self.shape[1:]) * self.dtype.itemsize

    def __getitem__(self, key):
        if isinstance(key, tuple) and len(key) == 1:
            key = key[0]
        if isinstance(key, slice) and self.shape:
            a, b, step = key.indices(self.shape[0])
            if step == 1:
                b = max(a, b)
                return ndarray(self.st, self.off + a * self._row_bytes(), self.dtype, (b - a,) + self.shape[1:])
        elif isinstance(key, (int, np.integer)) and self.shape:
            i = int(key) + (self.shape[0] if key < 0 else 0)
            if not 0 <= i < self.shape[0]:
                raise IndexError("index out of range")
            return ndarray(self.st, self.off + i * self._row_bytes(), self.dtype, self.shape[1:])
        elif key is Ellipsis:
            return self
        elif isinstance(key, ndarray) and key.dtype.kind in "iu" and self.shape and self._big_dev():
            rows = self.dev_in().view(-1, max(self._row_bytes(), 1))
            idx = torch.from_numpy(key._h().astype(np.int64).reshape(-1)).to(rows.device)
            out = empty((idx.numel(),) + self.shape[1:], self.dtype)
            out.dev_out().view(-1, max(self._row_bytes(), 1)).copy_(rows.index_select(0, idx))
            return out
        r = self._h()[_host_key(key)]
        return _wrap(np.array(r, copy=True)) if isinstance(r, np.ndarray) else _wrap(np.asarray(r))

    def __setitem__(self, key, value):
        if isinstance(key, tuple) and len(key) == 1:
            key = key[0]
        if (isinstance(key, slice) or key is Ellipsis) and self.shape:
            dst = self if key is Ellipsis else self[key] if (key.step in (None, 1)) else None
            if dst is not None and dst._assign(value):
                return
        elif isinstance(key, ndarray) and key.dtype.kind in "iu" and isinstance(value, ndarray) and self._big_dev():
            rows = self.dev_inout().view(-1, max(self._row_bytes(), 1))
            idx = torch.from_numpy(key._h().astype(np.int64).reshape(-1)).to(rows.device)
            rows.index_copy_(0, idx, value.dev_in().view(-1, max(self._row_bytes(), 1)))
            return
        self._hw()[_host_key(key)] = _host(value)

    def _assign(self, value):
        """self[...] = value without leaving the device, where that is where the data is -> done?"""
        n = self.nbytes
        if isinstance(value, ndarray):
            if value.dtype != self.dtype or value.size != self.size:
                return False
            if self._big_dev() or value.st.on_dev:
                self.dev_out().copy_(value.dev_in())
                return True
            return False
        if isinstance(value, np.ndarray):
            if value.dtype != self.dtype or value.size != self.size or not (self._big_dev() or n >= _BIG):
                return False
            xfer.h2d(self.dev_out(), np.ascontiguousarray(value).reshape(-1).view(np.uint8))
            STATS["h2d"] += n
            return True
        if isinstance(value, (int, np.integer)) and int(value) == 0 and self._big_dev():
            self.dev_out().zero_()
            return True
        return False

    # ---- transfers -----------------------------------------------------------------------------------------
    def get(self, stream=None, order="C", out=None, blocking=True):
        if out is None:
            out = np.empty(self.shape, self.dtype)
        if out.size != self.size or out.dtype.itemsize != self.dtype.itemsize:
            raise ValueError("get(out=): size mismatch")
        if not self.nbytes:
            return out
        if self.st.hv:
            np.copyto(out.reshape(-1).view(np.uint8), self._h().reshape(-1).view(np.uint8))
        else:
            flat = out.reshape(-1).view(np.uint8) if out.flags.c_contiguous else None
            if flat is None:
                out[...] = self._h()
            else:
                xfer.d2h(flat, self.dev_in())
                STATS["d2h"] += self.nbytes
        return out

    def set(self, arr, stream=None):
        arr = np.asarray(arr)
        if arr.size != self.size:
            raise ValueError("set(): size mismatch")
        if arr.dtype != self.dtype:
            arr = arr.astype(self.dtype)
        if not self._assign(arr):
            self._hw()[...] = arr.reshape(self.shape)

    def tobytes(self):
        return self.get().tobytes()

    def item(self):
        return self._h().item()

    def tolist(self):
        return self._h().tolist()

    def copy(self):
        out = empty(self.shape, self.dtype)
        if self.st.hv or not self.nbytes:
            out._hw()[...] = self._h()
        else:
            out.dev_out().copy_(self.dev_in())
        return out

    def astype(self, dtype, copy=True):
        dt = np.dtype(dtype)
        if dt == self.dtype:
            return self.copy() if copy else self
        return _wrap(self._h().astype(dt))

    def fill(self, v):
        if not self._assign(v):
            self._hw().fill(v)

    # ---- scalars -------------------------------------------------------------------------------------------
    def __int__(self):
        return int(self._h())

    def __float__(self):
        return float(self._h())

    def __bool__(self):
        return bool(self._h())

    def __index__(self):
        return int(self._h())

    def __repr__(self):
        where = "device" if self.st.on_dev else "host" if self.st.hv else "unset"
        return f"<refbind ndarray {self.shape} {self.dtype} {where}>"

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    # ---- everything else: NumPy on the host copy ----------------------------------------------------------------
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        f = getattr(np.ndarray, name, None)
        if f is None or not callable(f):
            raise AttributeError(name)
        return lambda *a, **kw: _host_call(getattr(self._h(), name), name, a, kw)


def _binop(name):
    def f(self, other):
        return _host_call(getattr(self._h(), name), name, (other,), {})
    return f


def _inplace(name):
    def f(self, other):
        getattr(self._hw(), name)(_host(other))
        return self
    return f


def _unop(name):
    def f(self):
        return _host_call(getattr(self._h(), name), name, (), {})
    return f


for _n in ("add", "sub", "mul", "truediv", "floordiv", "mod", "pow", "and", "or", "xor", "lshift", "rshift",
           "lt", "le", "gt", "ge", "eq", "ne", "matmul"):
    setattr(ndarray, f"__{_n}__", _binop(f"__{_n}__"))
    if _n not in ("lt", "le", "gt", "ge", "eq", "ne"):
        setattr(ndarray, f"__r{_n}__", _binop(f"__r{_n}__"))
        setattr(ndarray, f"__i{_n}__", _inplace(f"__i{_n}__"))
for _n in ("neg", "invert", "abs", "pos"):
    setattr(ndarray, f"__{_n}__", _unop(f"__{_n}__"))
ndarray.__hash__ = None


def _host(x):
    """shim arrays inside x (lists and tuples searched) -> NumPy views of their host copies"""
    if isinstance(x, ndarray):
        return x._h()
    if isinstance(x, tuple):
        return tuple(_host(v) for v in x)
    if isinstance(x, list):
        return [_host(v) for v in x]
    return x


_host_key = _host


def _wrap(r, inputs=()):
    """a NumPy result -> host-resident shim array (copied if it shares memory with an operand)"""
    if isinstance(r, np.generic):
        r = np.asarray(r)
    if isinstance(r, np.ndarray):
        if r.base is not None or not r.flags.c_contiguous or not r.flags.owndata:
            r = np.array(r, order="C", copy=True)
        st = _Storage(r.nbytes)
        st.host = r.reshape(-1).view(np.uint8) if r.size else np.empty(0, np.uint8)
        st.hv = True
        return ndarray(st, 0, r.dtype, r.shape)
    if isinstance(r, tuple):
        return tuple(_wrap(v) for v in r)
    if isinstance(r, list):
        return [_wrap(v) for v in r]
    return r


_STABLE = {"argsort", "sort"}


def _host_call(f, name, args, kw):
    STATS["host_ops"] += 1
    if name in _STABLE:
        kw = dict(kw)
        kw.pop("stable", None)
        kw["kind"] = "stable"            # CuPy sorts stably (seedpack/cpu.py:47-52)
    if _DEBUG:
        big = [a.nbytes for a in args if isinstance(a, ndarray) and a.nbytes >= (64 << 20)]
        if big:
            print(f"[refbind] {name} on the host over {sum(big) >> 20} MiB", flush=True)
    return _wrap(f(*_host(list(args)), **{k: _host(v) for k, v in kw.items()}))


# ---- creation ---------------------------------------------------------------------------------------------------
def _shape(shape):
    return (int(shape),) if isinstance(shape, (int, np.integer)) else tuple(int(s) for s in shape)


def empty(shape, dtype=float, order="C"):
    shape, dt = _shape(shape), np.dtype(dtype)
    return ndarray(_Storage(_prod(shape) * dt.itemsize), 0, dt, shape)


def zeros(shape, dtype=float, order="C"):
    shape, dt = _shape(shape), np.dtype(dtype)
    return ndarray(_Storage(_prod(shape) * dt.itemsize, zero=True), 0, dt, shape)


def full(shape, fill_value, dtype=None):
    return _wrap(np.full(_shape(shape), fill_value, dtype))


def empty_like(a, dtype=None):
    return empty(a.shape, dtype or a.dtype)


def zeros_like(a, dtype=None):
    return zeros(a.shape, dtype or a.dtype)


def asarray(a, dtype=None, order=None, blocking=False):
    if isinstance(a, ndarray):
        return a if dtype is None or a.dtype == np.dtype(dtype) else a.astype(dtype)
    if isinstance(a, np.ndarray) and a.nbytes >= _BIG and a.flags.c_contiguous and (dtype is None or a.dtype == np.dtype(dtype)):
        out = empty(a.shape, a.dtype)                # (copied to the device before this returns: no host copy first)
        out.set(a)
        return out
    h = np.array(a, dtype=dtype, order="C", copy=True)
    if h.nbytes >= _BIG:
        out = empty(h.shape, h.dtype)
        out.set(h)
        return out
    return _wrap(h)


array = asarray


def ascontiguousarray(a, dtype=None):
    return asarray(a, dtype)


def asnumpy(a, stream=None, order="C", out=None, blocking=True):
    if isinstance(a, ndarray):
        return a.get(out=out)
    if out is not None:
        np.copyto(out, a)
        return out
    return np.asarray(a, order=order)


def concatenate(arrs, axis=0, out=None, dtype=None):
    arrs = list(arrs)
    if axis == 0 and dtype is None and out is None and arrs and all(isinstance(a, ndarray) for a in arrs) \
            and any(a._big_dev() for a in arrs) and len({(a.dtype, a.shape[1:]) for a in arrs}) == 1:
        res = empty((sum(a.shape[0] for a in arrs),) + arrs[0].shape[1:], arrs[0].dtype)
        d, o = res.dev_out(), 0
        for a in arrs:
            d[o:o + a.nbytes].copy_(a.dev_in()); o += a.nbytes
        return res
    return _host_call(np.concatenate, "concatenate", (arrs,), dict(axis=axis))


def argsort(a, axis=-1, kind=None):
    return _host_call(np.argsort, "argsort", (a,), dict(axis=axis))


def sort(a, axis=-1, kind=None):
    return _host_call(np.sort, "sort", (a,), dict(axis=axis))


def __getattr__(name):
    """everything else is NumPy's: types, constants and ufunc objects as they are, functions on host copies"""
    a = getattr(np, name)
    if isinstance(a, type) or not callable(a):
        return a
    return lambda *args, **kw: _host_call(a, name, args, kw)


class _NS(types.SimpleNamespace):
    pass


random = _NS(RandomState=lambda seed=None: _RandomState(seed))
linalg = _NS(**{n: (lambda *a, _f=getattr(np.linalg, n), _n=n, **kw: _host_call(_f, _n, a, kw))
                for n in ("solve", "norm", "inv", "lstsq")})


class _RandomState:
    def __init__(self, seed=None):
        self._r = np.random.RandomState(seed)

    def __getattr__(self, name):
        f = getattr(self._r, name)
        return lambda *a, **kw: _host_call(f, name, a, kw)


# ---- runtime, devices, streams, pools ---------------------------------------------------------------------------------
class CUDARuntimeError(RuntimeError):
    pass


_MEMINFO = [0.0, None]


def _mem_get_info():
    """(free, total) device bytes; the driver call behind it synchronises, and the reference polls it in inner loops
    (repo3._dev_free, _fits_gpu, _window_bytes), so an answer is reused for a quarter of a second"""
    import time
    now = time.monotonic()
    if _MEMINFO[1] is None or now - _MEMINFO[0] > 0.25:
        _MEMINFO[0], _MEMINFO[1] = now, torch.cuda.mem_get_info(device_index())
    return _MEMINFO[1]


def _memcpy(dst, src, size, kind=None):
    raise NotImplementedError("raw memcpy is not part of this binding")


runtime = _NS(memGetInfo=_mem_get_info, CUDARuntimeError=CUDARuntimeError, getDeviceCount=torch.cuda.device_count,
              memcpy=_memcpy, deviceSetLimit=lambda *a: None, deviceSynchronize=lambda: torch.cuda.synchronize(device_index()))


class Device:
    def __init__(self, device=None):
        self.id = device_index() if device is None else int(device)

    @property
    def compute_capability(self):
        major, minor = torch.cuda.get_device_capability(self.id)
        return f"{major}{minor}"

    def synchronize(self):
        torch.cuda.synchronize(self.id)

    @property
    def mem_info(self):
        return torch.cuda.mem_get_info(self.id)

    def use(self):
        torch.cuda.set_device(self.id)
        return self

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class Stream:
    null = None

    def __init__(self, null=False, non_blocking=False, ptds=False):
        self.ptr = 0

    def synchronize(self):
        torch.cuda.current_stream(device_index()).synchronize()

    def use(self):
        return self

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


Stream.null = Stream(null=True)


class Event:
    def __init__(self, *a, **kw):
        self._e = torch.cuda.Event()

    def record(self, stream=None):
        self._e.record()

    def synchronize(self):
        self._e.synchronize()


cuda = _NS(runtime=runtime, Device=Device, Stream=Stream, Event=Event, get_current_stream=lambda: Stream.null,
           memory=_NS(OutOfMemoryError=torch.cuda.OutOfMemoryError))


class _DevicePool:
    """torch's caching allocator seen as CuPy's pool.  Cached blocks are handed back only when the cache has grown past
    half of the card: returning them costs a device-wide synchronisation (and so does asking the driver how much is
    free), and the reference asks for it after every file and every batch (repo3._release, _trim_cached)"""
    _limit = None

    def free_bytes(self):
        d = device_index()
        return max(0, torch.cuda.memory_reserved(d) - torch.cuda.memory_allocated(d))

    def used_bytes(self):
        return torch.cuda.memory_allocated(device_index())

    def total_bytes(self):
        return torch.cuda.memory_reserved(device_index())

    def n_free_blocks(self):
        return 0

    def free_all_blocks(self, stream=None):
        d = device_index()
        if self._limit is None:
            type(self)._limit = torch.cuda.get_device_properties(d).total_memory // 2
        if torch.cuda.memory_reserved(d) > self._limit:
            torch.cuda.empty_cache()

    def set_limit(self, size=None, fraction=None):
        pass


class _PinnedPool:
    """page-locked staging buffers, kept and reused by size class: locking pages is slow"""

    def __init__(self):
        self.free, self.lock, self.held, self.roots = {}, threading.RLock(), 0, {}      # (re-entrant: _give is a finalizer)

    @staticmethod
    def size_class(n):
        """n rounded up to an eighth of its power of two (at least 64 KiB): at most 12.5 % of a block is unused"""
        n = max(int(n), 1 << 16)
        step = max(1 << 13, (1 << (n - 1).bit_length()) >> 3)
        return -(-n // step) * step

    def owns(self, a):
        """whether NumPy array a is a block of this pool (not a view of one)"""
        return id(a) in self.roots

    def take(self, n):
        cls = self.size_class(n)
        with self.lock:
            lst = self.free.get(cls)
            t = lst.pop() if lst else None
        if t is None:
            try:
                t = torch.empty(cls, dtype=torch.uint8, pin_memory=True)
            except RuntimeError as e:
                raise CUDARuntimeError(str(e))
        a = t.numpy()
        self.roots[id(a)] = True
        weakref.finalize(a, self._give, cls, t, id(a))
        return a

    def _give(self, cls, t, key):
        with self.lock:
            self.roots.pop(key, None)
            self.free.setdefault(cls, []).append(t)

    def free_all_blocks(self, stream=None):
        with self.lock:
            self.free.clear()

    def n_free_blocks(self):
        return sum(len(v) for v in self.free.values())


_POOL, _PINNED = _DevicePool(), _PinnedPool()


def get_default_memory_pool():
    return _POOL


def get_default_pinned_memory_pool():
    return _PINNED


def empty_pinned(shape, dtype=float, order="C"):
    shape, dt = _shape(shape), np.dtype(dtype)
    n = _prod(shape) * dt.itemsize
    return _PINNED.take(n)[:n].view(dt).reshape(shape)


def zeros_pinned(shape, dtype=float, order="C"):
    a = empty_pinned(shape, dtype)
    a[...] = 0
    return a


cupyx = types.ModuleType("cupyx")
cupyx.empty_pinned, cupyx.zeros_pinned = empty_pinned, zeros_pinned


# ---- kernels --------------------------------------------------------------------------------------------------------
class RawModule:
    """nothing is compiled: a function is the C-ABI binding of the reference kernel of that name"""

    def __init__(self, code=None, path=None, options=(), **kw):
        # the integer #defines of the reference's source: switches its modules are compiled with (SIGN, RANK, SEGA ...),
        # which the bindings hand to the library as run-time arguments
        import re
        self.defines = {k: int(v) for k, v in re.findall(r"^#define[ \t]+(\w+)[ \t]+(-?\d+)[ \t]*(?://.*)?$", code or "", re.M)}

    def get_function(self, name):
        from . import kernels
        return kernels.function(name, self.defines)

    def get_global(self, name):
        raise NotImplementedError(f"device global {name}: the reference's modules are not loaded here")


def ElementwiseKernel(in_params, out_params, operation, name="kernel", **kw):
    from . import kernels
    return kernels.elementwise(name)
