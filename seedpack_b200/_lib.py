"""ctypes binding of libseedgrow.so (the C ABI declared in include/seedgrow.h).

There is no fallback: if the shared object is missing or a call fails, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libseedgrow.so")

DT_BF16, DT_F16, DT_F32 = 0, 1, 2


class SgError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = lib().sg_status_string(status).decode()
        if status == 8:
            msg += " (" + lib().sg_last_cuda_error().decode() + ")"
        super().__init__(f"{where}: {msg} [status {status}]")


class sg_tensor(ctypes.Structure):
    _fields_ = [("x_off", ctypes.c_int64), ("y_off", ctypes.c_int64), ("w_off", ctypes.c_int64),
                ("n_rows", ctypes.c_int64), ("n_per_row", ctypes.c_int64)]


_lib = None

# name -> (restype, argtypes); every symbol include/seedgrow.h declares
_P, _I, _Z, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64
SIGNATURES = {
    "sg_version": (_I, []),
    "sg_status_string": (ctypes.c_char_p, [_I]),
    "sg_last_cuda_error": (ctypes.c_char_p, []),
    "sg_type_info": (_I, [_I, ctypes.POINTER(_I), ctypes.POINTER(_I)]),
    "sg_type_needs_imatrix": (_I, [_I]),
    "sg_status_fetch": (_I, [_I, _P, ctypes.POINTER(_I)]),
    "sg_tables_install": (_I, [_I, _P]),
    "sg_tables_host": (_I, [_I, _I, ctypes.POINTER(_P), ctypes.POINTER(_Z)]),
    "sg_quantize_scratch_bytes": (_Z, [_I, ctypes.POINTER(sg_tensor), _I]),
    "sg_quantize_tensors": (_I, [_I, _P, _I, _I, _P, _I, _P, _P, ctypes.POINTER(sg_tensor), _I, _P, _Z]),
    "sg_dequantize": (_I, [_I, _P, _I, _P, _P, _L]),
    "sg_convert_float": (_I, [_I, _P, _P, _I, _P, _I, _L]),
    "sg_residual_xor": (_I, [_I, _P, _P, _P, _P, _P, _Z, _P]),
    "sg_residual_blocks": (_I, [_I, _P, _P, _P, _I, _L, _P, _P]),
    "sg_rans_hist": (_I, [_I, _P, _P, _P, _I, _L, _P]),
    "sg_rans_tables": (_I, [_I, _P, _P, _I, _I, _P, _P]),
    "sg_rans_encode": (_I, [_I, _P, _P, _P, _I, _L, _I, _I, _P, _P, _Z, _P]),
    "sg_scan_gather": (_I, [_I, _P, _P, _Z, _P, _I, _P, ctypes.c_uint64, _P]),
    "sg_rans_decode": (_I, [_I, _P, _P, _P, _P, _I, _L, _I, _I, _P, _P, _I, _P]),
    "sg_qr_hist": (_I, [_I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I]),
    "sg_qr_encode": (_I, [_I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _Z, _P, _I]),
    "sg_qr_decode": (_I, [_I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I]),
    "sg_qr_stage_bytes": (_Z, [_I, _L]),
    "sg_qr_stage": (_I, [_I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _L, _P, _Z]),
    "sg_qr_stage_hist": (_I, [_I, _P, _I, _L, _P, _P]),
    "sg_qr_stage_encode": (_I, [_I, _P, _I, _L, _P, _P, _I, _P, _P, _Z, _P]),
    "sg_r2_hist": (_I, [_I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P]),
    "sg_r2_encode": (_I, [_I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _Z, _P]),
    "sg_r2_decode": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P]),
    "sg_row_hash": (_I, [_I, _P, _P, _I, _I, _P]),
    "sg_copy_rows": (_I, [_I, _P, _P, _I, _P, _I]),
    "sg_r2_stats_scratch_bytes": (_Z, [_I, _I]),
    "sg_r2_stats": (_I, [_I, _P, _P, _I, _I, _P, _P, _P, _P, _Z]),
    "sg_dm_log2": (_I, [_I, _P, _P, _L, _P]),
    "sg_dm_exp2": (_I, [_I, _P, _P, _L, _P]),
    "sg_dm_rows": (_I, [_I, _P, _P, _L, _L, _I, _P]),
    "sg_dm_cols": (_I, [_I, _P, _P, _L, _L, _I, _P, _P]),
    "sg_qr_block_fields": (_I, [_I, _P, _I, _P, _L, _P]),
    "sg_qr_blocks_from_fields": (_I, [_I, _P, _I, _P, _I, _P]),
    "sg_qr_intervals": (_I, [_I, _P, _I, _P, _L, _P, _P]),
    "sg_qr_weight_equal": (_I, [_I, _P, _I, _P, _P, _L, _P]),
    "sg_qr_grid_half_step": (_I, [_I, _P, _I, _P, _L, _P]),
    "sg_m6_hist": (_I, [_I, _P, _P, _P, _P, _P, _I, _P, _I, _P]),
    "sg_m6_encode": (_I, [_I, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _Z, _P]),
    "sg_m6_decode": (_I, [_I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _P]),
    "sg_rans_chain_encode": (_I, [_I, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P]),
    "sg_rans_chain_decode": (_I, [_I, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P]),
    "sg_m21_hist_a": (_I, [_I, _P] + [_P] * 4 + [_I, _I] + [_P] * 5 + [_I, _I, _P]),
    "sg_m21_encode_a": (_I, [_I, _P] + [_P] * 4 + [_I, _I] + [_P] * 5 + [_I, _I, _P, _P, _Z, _P]),
    "sg_m21_decode_a": (_I, [_I, _P] + [_P] * 5 + [_I, _I] + [_P] * 5 + [_I, _I, _P, _P, _P, _P]),
    "sg_m21_hist_b": (_I, [_I, _P] + [_P] * 4 + [_I, _I] + [_P] * 3 + [_I, _I, _I, _I, _P]),
    "sg_m21_encode_b": (_I, [_I, _P] + [_P] * 4 + [_I, _I] + [_P] * 3 + [_I, _I, _I, _P, _P, _Z, _P]),
    "sg_m21_decode_b": (_I, [_I, _P] + [_P] * 5 + [_I, _I] + [_P] * 3 + [_I, _I, _I, _P, _P, _P, _P]),
    "sg_m21_predict": (_I, [_I, _P, _P, _I, _I, _I, _P, _I, _P, _P, _I, _P, _P]),
    "sg_m21_predict_multi": (_I, [_I, _P, _P, _P, _P, _I, _I] + [_P] * 7 + [_I, _P, _P]),
    "sg_m21_hist_c": (_I, [_I, _P] + [_P] * 8 + [_I] + [_P] * 6 + [_I, _P]),
    "sg_m21_encode_c": (_I, [_I, _P] + [_P] * 8 + [_I] + [_P] * 6 + [_I, _P, _P, _Z, _P]),
    "sg_m21_decode_c": (_I, [_I, _P, _P, _P, _P, _I] + [_P] * 7 + [_I] + [_P] * 6 + [_I, _P, _P, _P]),
    "sg_sib_half_step": (_I, [_I, _P, _P, _P, _P, _L, _P]),
    "sg_sib_est_add": (_I, [_I, _P, _P, _P, _L, _P, _P]),
    "sg_sib_est_seed": (_I, [_I, _P, _P, _P, _P, _L, _P]),
    "sg_m24_hist": (_I, [_I, _P, _P, _P, _P, _I, _P, _P, _P, _P]),
    "sg_m24_encode": (_I, [_I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _Z, _P]),
    "sg_m24_decode": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P]),
    "sg_dm_rows_f64": (_I, [_I, _P, _P, _L, _L, _I, _P]),
    "sg_dm_gram": (_I, [_I, _P, _P, _L, _I, _L, _P]),
    "sg_dm_bdot": (_I, [_I, _P, _P, _P, _L, _I, _L, _P]),
    "sg_dm_solve": (_I, [_I, _P, _P, _P, _L, _I, _P]),
    "sg_selftest_nearest_int": (_I, [_I, _P, _P, _P, _L]),
    "sg_quantize_legacy_imx_static": (_I, [_I, _P, _I, _P, _I, _P, _P, ctypes.POINTER(sg_tensor), _I]),
}


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m seedpack_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def check(status, where):
    if status != 0:
        raise SgError(status, where)


# ---- optional per-call device timing and copy accounting (benchmarks) ----------------------------------------------
import contextlib
import threading

_TIMES = None
_TLOCK = threading.Lock()
COPIES = {"h2d": 0, "d2h": 0}          # bytes the host-side classes moved between host and device


def count_h2d(n):
    COPIES["h2d"] += int(n)


def count_d2h(n):
    COPIES["d2h"] += int(n)


@contextlib.contextmanager
def timed(name):
    """with timing_start() active: CUDA-event time of the enclosed launches on torch's current stream, summed per name
    (not while timing_start(calls=True) times every library call itself)"""
    if _TIMES is None or "__calls__" in _TIMES:
        yield
        return
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    yield
    e1.record()
    _TIMES.setdefault(name, []).append((e0, e1))


def _label(name, args):
    if name == "sg_quantize_tensors":
        return f"{name}[{args[2]}{'' if args[7] is None else '+imx'}]"
    if name in ("sg_qr_hist", "sg_qr_encode", "sg_qr_decode", "sg_qr_stage", "sg_qr_stage_hist", "sg_qr_stage_encode", "sg_dequantize"):
        return f"{name}[{args[2]}]"
    return name


def timing_start(calls=False):
    """start collecting device times.  calls=True: every library call that takes a stream is timed by its entry-point
    name (quantisers and QR calls by type as well) with a pair of CUDA events recorded around it on torch's current
    stream; the calls of different host threads are serialised while this is on, so that no pair spans another
    thread's launches.  calls=False: only the regions marked with timed() in the host classes"""
    global _TIMES
    _TIMES = {}
    if not calls:
        return
    import torch
    L = lib()
    _TIMES["__calls__"] = {}
    for name, (res, args) in SIGNATURES.items():
        if len(args) < 2 or args[0] is not _I or args[1] is not _P or name in ("sg_status_fetch", "sg_tables_install"):
            continue
        raw = getattr(L, name)

        def wrapped(*a, _raw=raw, _name=name):
            with _TLOCK:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                rc = _raw(*a)
                e1.record()
                _TIMES.setdefault(_label(_name, a), []).append((e0, e1))
            return rc
        _TIMES["__calls__"][name] = raw
        setattr(L, name, wrapped)


def timing_stop(counts=False):
    """-> {name: milliseconds} of everything timed since timing_start() (with counts: {name: (ms, calls)})"""
    global _TIMES
    import torch
    torch.cuda.synchronize()
    t = _TIMES or {}
    for name, raw in (t.pop("__calls__", None) or {}).items():
        setattr(lib(), name, raw)
    out = {k: (sum(a.elapsed_time(b) for a, b in v), len(v)) for k, v in t.items()}
    _TIMES = None
    return out if counts else {k: v[0] for k, v in out.items()}
