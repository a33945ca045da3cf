"""Binding of the reference's host code to libseedgrow.so.

The reference keeps its command line, repository logic, windowing and container in Python and reaches the GPU
through CuPy (seedpack/xp.py).  `install()` puts this package's realisation of that layer underneath it:

    cupy / cupyx            -> refbind.cupy_shim   (device arrays, launches, pools: seedpack/xp.py:6-18)
    zstandard               -> seedpack_b200.zstd  (only where the zstandard package is not installed)
    gpuquant.GPUQuant       -> refbind.quant.GPUQuant          (seedpack/gpuquant.py:285-456)
    gpuquant.to_host        -> refbind.quant.to_host           (gpuquant.py:262-282)
    qr.encode / qr.decode   -> seedpack_b200.qr.QRCodec        (seedpack/qr.py:1007-1090; model once per block)
    BF16v2._stats           -> sg_r2_stats                     (seedpack/bf16v2.py:225-244)
    M28RepoGPU._float_dev   -> sg_convert_float                (seedpack/repo3.py:673-689)
    every RawModule kernel  -> refbind.kernels                 (R2, detmath, gather, single-pass QR, dequantisers)
    cpukernels.RawModule    -> raises                          (the reference's CUDA source is never compiled)

After that `seedpack.cli.main()` - or `python -m seedpack_b200.refbind pack|unpack|test|list ...` - is the reference's
own program with every kernel served by this library.  The reference is found as an installed / importable
`seedpack` package, under $SEEDPACK_REFERENCE, or in baseline/_ref of this tree.
"""
import importlib
import importlib.util
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_state = {}


def find_reference():
    """directory that holds the reference's `seedpack` package, or None"""
    cands = [os.environ.get("SEEDPACK_REFERENCE"), os.path.join(_ROOT, "baseline", "_ref")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "seedpack", "repo3.py")):
            return c
    spec = importlib.util.find_spec("seedpack")
    if spec is not None and spec.origin:
        return os.path.dirname(os.path.dirname(spec.origin))
    return None


def available():
    return find_reference() is not None


def install(reference=None, staged_qr=None):
    """bind the reference (see the module docstring) -> its `seedpack` package.  Idempotent.
    staged_qr False (or SEEDGROW_QR_SINGLE_PASS=1): qr.encode / qr.decode stay the reference's functions and their
    qr_hist / qr_enc / qr_dec launches go through the one-to-one kernel bindings (same bytes, the model run twice)"""
    if staged_qr is None:
        staged_qr = os.environ.get("SEEDGROW_QR_SINGLE_PASS") != "1"
    if "pkg" in _state:
        return _state["pkg"]
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("seedpack_b200.refbind needs a CUDA device: there is no CPU path (the reference has --cpu)")
    if os.environ.get("SEEDPACK_CPU") == "1":
        raise RuntimeError("SEEDPACK_CPU=1 selects the reference's own CPU kernels; unset it to bind libseedgrow.so")
    if "seedpack" in sys.modules:
        raise RuntimeError("the reference was imported before refbind.install()")
    ref = reference or find_reference()
    if ref is None:
        raise RuntimeError("the reference package `seedpack` was not found (install it, or set SEEDPACK_REFERENCE)")
    from .. import _lib
    _lib.lib()                                    # fails loudly if the CUDA library is not built
    from . import cupy_shim, kernels, quant
    cupy_shim.bind_device()                       # this process's GPU: the one current now, for all of its threads
    sys.modules["cupy"] = cupy_shim
    sys.modules["cupyx"] = cupy_shim.cupyx
    if importlib.util.find_spec("zstandard") is None:
        from .. import zstd
        sys.modules["zstandard"] = zstd
    if ref not in sys.path:
        sys.path.insert(0, ref)
    import seedpack
    from seedpack import cpukernels, xp
    if xp.CPU or xp.cp is not cupy_shim:
        raise RuntimeError("the reference did not pick up the binding's array module")

    def _no_cpu_kernels(*a, **kw):
        raise RuntimeError("the reference's CUDA source is not compiled in this process: kernels come from libseedgrow.so")
    cpukernels.RawModule = _no_cpu_kernels
    from seedpack import bf16v2, gpuquant, qr, repo3
    gpuquant.GPUQuant = repo3.GPUQuant = quant.GPUQuant
    gpuquant.to_host = repo3.to_host = quant.to_host
    qr._GQ = None
    _bind_qr(qr, staged_qr)
    _bind_r2(bf16v2)
    _bind_float(repo3)
    _bind_residual(repo3)
    from seedpack import rans
    _bind_rans(rans)
    from seedpack import detmath, gpu3
    from . import plan
    gpu3.GPU3._row_matrix = plan.row_matrix       # M21's row planner: device twins of two chains of array operations
    gpu3.GPU3._plan_tensor = plan.make(detmath)
    _state["pkg"] = seedpack
    return seedpack


# ---- QR ---------------------------------------------------------------------------------------------------------------
def _bind_qr(qr, staged):
    """qr.encode / qr.decode through QRCodec: the model of a block is run once (sg_qr_stage*), where the reference's
    kernels - and their one-to-one bindings in refbind.kernels - run it in the histogram and again in the coder"""
    import numpy as np
    import torch
    from .. import qr as own
    from . import cupy_shim as cp
    from . import twins
    from .quant import from_torch
    if not staged:
        return
    codecs = {}

    def codec():
        d = cp.device_index()
        if d not in codecs:
            codecs[d] = own.QRCodec(d, staged=True)
        return codecs[d]

    def arr(a):
        """host or device bytes of a tensor as QRCodec takes them; a host array whose bytes are on the device already
        (refbind.twins) is taken from there"""
        if isinstance(a, cp.ndarray):
            return a.dev_in()
        t = twins.find(a)
        return a if t is None else t

    def encode(T, items, seed_dev, imx_dev=None, mv=None):
        its = [(arr(it[0]), arr(it[1])) + tuple(it[2:]) for it in items]
        return codec().encode(T, its, arr(seed_dev), None if imx_dev is None else arr(imx_dev).view(torch.float32), mv)

    def decode(T, buf, items, seed_dev, imx_dev=None):
        its = [(arr(it[0]),) + tuple(it[1:]) for it in items]
        F = codec().decode(T, buf, its, arr(seed_dev), None if imx_dev is None else arr(imx_dev).view(torch.float32))
        return from_torch(F)

    encode.__doc__, decode.__doc__ = qr.encode.__doc__, qr.decode.__doc__
    qr.encode, qr.decode = encode, decode


# ---- R2 ---------------------------------------------------------------------------------------------------------------
def _bind_r2(bf16v2):
    """BF16v2 and R2Tensors stay the reference's classes; their kernels come from refbind.kernels.  The per-tensor
    statistics (`_stats`: a chain of array operations over the whole tensor around detmath) are one library call"""
    import ctypes
    import numpy as np
    import torch
    from .. import _lib
    from . import cupy_shim as cp

    def _stats(self, dev, rl):
        nr = dev.size // 2 // rl
        rfi, cfi, scl = cp.empty(nr, np.int16), cp.empty(rl, np.int16), cp.empty(rl, np.int8)
        L = _lib.lib()
        need = L.sg_r2_stats_scratch_bytes(nr, rl)
        scratch = torch.empty(need + 16, dtype=torch.uint8, device=dev.dev_in().device)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        d = cp.device_index()
        _lib.check(L.sg_r2_stats(d, ctypes.c_void_p(torch.cuda.current_stream(d).cuda_stream),
                                 p(dev.dev_in()), nr, rl, p(rfi.dev_out()), p(cfi.dev_out()), p(scl.dev_out()), p(scratch), need),
                   "sg_r2_stats")
        return rfi, cfi, scl

    bf16v2.BF16v2._stats = _stats


# ---- residual against the stored quant --------------------------------------------------------------------------------
def _bind_residual(repo3):
    """The comparisons of a stored tensor with its prediction (repo3.py:476-497: `_diff_async`, `_count_diff`) on the
    device (sg_residual_xor, counting only).  The reference compares on the host, in 2 MiB chunks handed to a thread
    pool, after downloading every prediction.  Here the prediction is still on the device when its host copy arrives
    (refbind.quant._download registers it), and the span of the file that `_residual_tensors` works on is uploaded once,
    when it starts: each comparison is then one launch and one 8-byte read, and the QR coder later takes the same device
    bytes as its inputs.  Operands without a device copy go to the reference's own functions.  The in-place XOR of
    float tensors (`_xor_async`, `_xor3`) stays on the host: its result is wanted there, by zstd"""
    import numpy as np
    import torch
    from .. import residual
    from . import cupy_shim as cp
    from . import quant, twins, xfer
    ref_diff, ref_count, ref_tensors = repo3._diff_async, repo3._count_diff, repo3.M28RepoGPU._residual_tensors
    MIN_SPAN = 1 << 20

    class _Flag:
        """what `_diff_async` hands back: a future-like whose result is whether the device counter is non-zero; the
        counter is read when the result is asked for (repo3.py:1120 asks after all of a file's predictions are made),
        so the comparisons of a file queue up behind one another without a synchronisation each"""

        def __init__(self, counter):
            self.counter = counter

        def result(self, timeout=None):
            return int(self.counter.item()) > 0

        def done(self):
            return True

    def _pair(a, b):
        if b is None or not isinstance(a, np.ndarray) or not isinstance(b, np.ndarray) or a.nbytes != b.nbytes:
            return None, None
        da = twins.find(a)
        if da is None:
            return None, None
        db = twins.find(b)
        if db is None:
            return None, None
        cp.device_index()
        return da, db

    def _diff_async(r, p):
        da, db = _pair(r, p)
        if da is None:
            return ref_diff(r, p)
        return [_Flag(residual.count_diff(da, db, sync=False))]

    def _count_diff(a, b=None):
        da, db = _pair(a, b)
        if da is None:
            return ref_count(a, b)
        return residual.count_diff(da, db)

    def _residual_tensors(self, view, at, ts, held, memo=None, hashes=None):
        if isinstance(view, np.ndarray) and view.flags.c_contiguous and view.nbytes >= MIN_SPAN and any(k == "rq" for _, k in ts) \
                and twins.find(view[:1]) is None:
            d = cp.device_index()
            lead = int(at) % 16                 # tensors start on 32-byte file offsets: keep them 16-byte aligned on the device
            buf = torch.empty(view.nbytes + 16 + 64, dtype=torch.uint8, device=torch.device("cuda", d))
            dev = buf[lead:lead + view.nbytes]
            xfer.h2d(dev, view.reshape(-1).view(np.uint8))
            cp.STATS["h2d"] += view.nbytes
            twins.register(view, dev)
        return ref_tensors(self, view, at, ts, held, memo, hashes)

    repo3._diff_async, repo3._count_diff = _diff_async, _count_diff
    repo3.M28RepoGPU._residual_tensors = _residual_tensors
    repo3._pcopy = quant.pcopy(repo3._pcopy)


# ---- the scalar stream coder (rans.py) -------------------------------------------------------------------------------------
def _bind_rans(rans):
    """rans.encode / rans.decode (seedpack/rans.py:152-164: host arrays in, host bytes / symbols out; numba loops) run
    as one stream = one lane of sg_rans_chain_encode / sg_rans_chain_decode.  M22 (bf16codec.py) is their caller"""
    import ctypes
    import numpy as np
    import torch
    from .. import _lib
    from . import cupy_shim as cp
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def _setup(ctx, freqs):
        d = cp.device_index()
        dev = torch.device("cuda", d)
        st = ctypes.c_void_p(torch.cuda.current_stream(d).cuda_stream)
        f = np.ascontiguousarray(freqs, np.uint16)
        if f.ndim != 2 or f.shape[1] != 256:
            raise ValueError("rans: tables of 256 symbols expected")
        sums = f.sum(1, dtype=np.int64)
        if ((sums != 0) & (sums != rans.PROB_SCALE)).any():
            raise ValueError("coder tables: a row of frequencies does not sum to 2^PB (damaged table part)")
        c = np.ascontiguousarray(ctx)
        if c.dtype.kind not in "iu" or c.dtype.itemsize > 4:
            c = c.astype(np.int32)
        if c.size and (int(c.min()) < 0 or int(c.max()) >= f.shape[0]):
            raise ValueError("rans: a context outside the tables")
        ntab = f.shape[0]
        enc = torch.empty(ntab * 256 * 2, dtype=torch.int32, device=dev)
        lut = torch.zeros(ntab << rans.PROB_BITS, dtype=torch.uint8, device=dev)
        fd = torch.from_numpy(f.view(np.int16)).to(dev)
        _lib.check(_lib.lib().sg_rans_tables(d, st, p(fd), ntab, rans.PROB_BITS, p(enc), p(lut)), "sg_rans_tables")
        cd = torch.from_numpy(c.view(np.uint8).reshape(-1)).to(dev)
        _lib.count_h2d(f.nbytes + c.nbytes)
        return d, dev, st, ntab, enc, lut, cd, c.dtype.itemsize, (fd,)

    def encode(sym, ctx, freqs):
        s = np.ascontiguousarray(sym, np.uint8).reshape(-1)
        n = s.size
        d, dev, st, ntab, enc, lut, cd, cb, keep = _setup(ctx, freqs)
        cap = (2 * n + 16 + 15) // 16 * 16
        sd = torch.from_numpy(s).to(dev) if n else torch.zeros(16, dtype=torch.uint8, device=dev)
        slots = torch.empty(cap, dtype=torch.uint8, device=dev)
        offs = torch.tensor([0, n, 0, cap], dtype=torch.int64, device=dev)
        ln = torch.zeros(1, dtype=torch.int64, device=dev)
        _lib.check(_lib.lib().sg_rans_chain_encode(d, st, p(sd), p(cd) if n else p(sd), cb, p(offs), 1, ntab, p(enc), p(slots), p(offs[2:]), p(ln)),
                   "sg_rans_chain_encode")
        k = int(ln.item())
        if k == 0xfffffffe:
            raise ValueError("rANS encoder: a coded symbol has frequency 0 in its table")
        if k == 0xffffffff:
            raise ValueError("rANS encoder: the stream outgrew its slot")
        _lib.count_h2d(n); _lib.count_d2h(k)
        return slots[cap - k:].cpu().numpy().tobytes()

    def decode(buf, ctx, freqs):
        n = int(np.asarray(ctx).shape[0])
        b = np.frombuffer(buf, np.uint8)
        d, dev, st, ntab, enc, lut, cd, cb, keep = _setup(ctx, freqs)
        if n == 0:
            return np.empty(0, np.uint8)
        bd = torch.zeros(b.size + 16, dtype=torch.uint8, device=dev)
        bd[:b.size] = torch.from_numpy(b.copy()).to(dev)
        offs = torch.tensor([0, n, 0, b.size], dtype=torch.int64, device=dev)
        out = torch.empty(n, dtype=torch.uint8, device=dev)
        _lib.check(_lib.lib().sg_rans_chain_decode(d, st, p(bd), p(offs[2:]), p(offs[3:]), p(cd), cb, p(offs), 1, ntab, p(enc), p(lut), p(out), None),
                   "sg_rans_chain_decode")
        bits = ctypes.c_int(0)
        _lib.check(_lib.lib().sg_status_fetch(d, st, ctypes.byref(bits)), "sg_status_fetch")
        if bits.value & 4:
            raise ValueError("rans: corrupt coded stream")
        _lib.count_h2d(b.size); _lib.count_d2h(n)
        return out.cpu().numpy()

    rans.encode, rans.decode = encode, decode


# ---- float tensors -----------------------------------------------------------------------------------------------------
def _bind_float(repo3):
    import ctypes
    import numpy as np
    import torch
    from .. import _lib
    from . import cupy_shim as cp
    F32, F16, BF16 = repo3.F32, repo3.F16, repo3.BF16
    code = {BF16: (_lib.DT_BF16, 2), F16: (_lib.DT_F16, 2), F32: (_lib.DT_F32, 4)}
    reference_float_dev = repo3.M28RepoGPU._float_dev

    def _float_dev(self, bt, ttype, dev=None, lo=0, hi=None):
        a = self._src(bt, dev=dev)
        if bt.type not in code or not isinstance(a, cp.ndarray):
            return reference_float_dev(self, bt, ttype, dev, lo, hi)      # a quantised seed: dequantised first
        a = a[lo:hi]
        if bt.type == ttype:
            return a.view(np.uint8)
        (sd, _), (dd, dsz) = code[bt.type], code[ttype]
        y = cp.empty(a.size * dsz, np.uint8)
        src = a.dev_in()
        if src.data_ptr() % 16:
            src = src.clone()
        d = cp.device_index()
        _lib.check(_lib.lib().sg_convert_float(d, ctypes.c_void_p(torch.cuda.current_stream(d).cuda_stream),
                                               ctypes.c_void_p(src.data_ptr()), sd, ctypes.c_void_p(y.dev_out().data_ptr()), dd, a.size),
                   "sg_convert_float")
        return y

    repo3.M28RepoGPU._float_dev = _float_dev


def main(argv=None):
    """the reference's command line on the bound kernels"""
    install()
    from seedpack import cli
    if argv is not None:
        sys.argv = ["seedpack"] + list(argv)
    return cli.main()
