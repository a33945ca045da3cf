"""TEST TOOLING - run the reference's command line in a child process, in one of two ways:

    python tests/tools/refcli.py cpu  pack --cpu -o a.seedpack <dir>     the reference as it is (its own CPU kernels)
    python tests/tools/refcli.py emu  pack -o b.seedpack <dir>           the reference over seedpack_b200.refbind's array
                                                                        module with NO GPU: "device" memory is host memory
                                                                        and every launch runs the reference's CPU build of
                                                                        the kernel of that name

The second form checks the binding's array module (residency, views, slice assignment, host fall-backs) under the
whole of the reference's host code on a machine without a GPU: its archive must equal the first form's byte for
byte.  The C-ABI kernels themselves are not involved; the GPU tests cover those.
The reference is taken from $SEEDPACK_REFERENCE or baseline/_ref; zstandard, where missing, is seedpack_b200.zstd.
"""
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def _common():
    from seedpack_b200 import refbind
    ref = refbind.find_reference()
    if ref is None:
        sys.exit("reference package not found")
    sys.path.insert(0, ref)
    if importlib.util.find_spec("zstandard") is None:
        from seedpack_b200 import zstd
        sys.modules["zstandard"] = zstd
    os.environ.setdefault("SEEDPACK_CACHE", os.path.join(ROOT, "oracle", "_build", "refcache"))
    os.environ.setdefault("NUMBA_CACHE_DIR", os.path.join(ROOT, "oracle", "_build", "numba"))
    os.makedirs(os.environ["SEEDPACK_CACHE"], exist_ok=True)


def run_cpu(argv):
    _common()
    from seedpack.cli import main
    sys.argv = ["seedpack"] + argv
    main()


def run_emu(argv):
    _common()
    import numpy as np
    import torch
    from seedpack_b200.refbind import cupy_shim as cp
    cp._device = lambda: torch.device("cpu")
    cp._mem_get_info = lambda: (32 << 30, 64 << 30)
    cp.runtime.memGetInfo = cp._mem_get_info
    cp.runtime.getDeviceCount = lambda: 1
    cp.runtime.deviceSynchronize = lambda: None
    import ctypes
    cp.runtime.memcpy = lambda dst, src, size, kind=None: ctypes.memmove(dst, src, size)
    cp.Device.synchronize = lambda self: None
    cp.Device.__init__ = lambda self, device=None: setattr(self, "id", 0)
    cp.Device.compute_capability = "cpu"
    cp._DevicePool.free_bytes = lambda self: 0
    cp._DevicePool.used_bytes = lambda self: 0
    cp._DevicePool.total_bytes = lambda self: 0
    cp._DevicePool.free_all_blocks = lambda self, stream=None: None
    cp.ndarray.ctypes = property(lambda self: self._hw().ctypes)      # every array a CPU kernel touches may be written
    sys.modules["cupy"], sys.modules["cupyx"] = cp, cp.cupyx
    from seedpack import cpukernels, xp
    assert xp.cp is cp and not xp.CPU

    class EmuModule:
        def __init__(self, code=None, path=None, options=(), exact_division=False, **kw):
            self.m = cpukernels.RawModule(code=code, exact_division=exact_division)

        def get_function(self, name):
            return self.m.get_function(name)

        def get_global(self, name):
            return self.m.get_global(name)

    cp.RawModule = EmuModule

    def bf16_to_f32(a, y=None):
        r = (a._h().astype(np.uint32) << 16).view(np.float32)
        if y is None:
            return cp.asarray(r)
        y._hw()[...] = r
        return y
    cp.ElementwiseKernel = lambda *a, **kw: bf16_to_f32
    xp.ptr = lambda a: a._hw().ctypes.data
    xp.CPU = True                        # GPUQuant builds its CPU module (no NVRTC); arrays stay the binding's
    from seedpack import gpuquant
    gpuquant.xp.CPU = True
    # the binding's twin of M21's row planner (refbind/plan.py), here on CPU tensors over the reference's CPU detmath kernels
    from seedpack import detmath, gpu3
    from seedpack_b200.refbind import plan
    gpu3.GPU3._plan_tensor = plan.make(detmath)
    from seedpack.cli import main
    sys.argv = ["seedpack"] + argv
    main()
    print("shim stats:", cp.STATS, file=sys.stderr)


if __name__ == "__main__":
    {"cpu": run_cpu, "emu": run_emu}[sys.argv[1]](sys.argv[2:])
