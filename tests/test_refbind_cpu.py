"""The binding's array module under the reference's whole host program, on a machine without a GPU.

tests/tools/refcli.py runs the reference's command line twice on a seeded repository of a few megabytes: as it is
(`--cpu`, its own NumPy stand-in for CuPy and its own CPU build of its kernels), and over seedpack_b200.refbind's
CuPy stand-in with "device" memory redirected to host memory and launches redirected to that same CPU build.  The
second run exercises residency tracking, views, slice assignment, row gathers and the host fall-backs of
refbind/cupy_shim.py in every place the reference's pack and unpack paths touch an array; its archive must be the
first run's byte for byte, and each side must restore the other's archive.  (The C-ABI kernels are not involved
here; tests/test_archive_gpu.py does the same with them on the GPU.)
"""
import hashlib
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
TOOL = os.path.join(HERE, "tools", "refcli.py")


def _have_reference():
    from seedpack_b200 import refbind
    return refbind.available()


def _have_oracle():
    from oracle import ref
    return ref.available()


def run(mode, *args, cwd):
    env = dict(os.environ, SOURCE_DATE_EPOCH="1700000000")
    env.pop("SEEDPACK_CPU", None)
    r = subprocess.run([sys.executable, TOOL, mode, *args], cwd=cwd, env=env, capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r


def make_repo(root, config, seed=1):
    from oracle import ref
    from seedpack_b200 import synthrepo
    return synthrepo.make_repo(root, config, lambda ty, bits, w: ref.quantize(ty, ref.bf16_to_f32(bits), w), seed=seed)


def digest(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for b in iter(lambda: f.read(1 << 22), b""):
            h.update(b)
    return h.hexdigest()


def same_tree(a, b):
    names = sorted(os.listdir(a))
    assert names == sorted(os.listdir(b))
    for n in names:
        assert digest(os.path.join(a, n)) == digest(os.path.join(b, n)), n


@pytest.mark.skipif(not (_have_reference() and _have_oracle()), reason="needs the reference package (baseline/_ref or "
                    "$SEEDPACK_REFERENCE) and oracle/_ref")
def test_reference_over_the_array_module_gives_the_reference_archive(tmp_path):
    repo = str(tmp_path / "repo")
    make_repo(repo, "c1-nano")
    a, b = str(tmp_path / "cpu.seedpack"), str(tmp_path / "emu.seedpack")
    run("cpu", "pack", "--cpu", "-q", "-o", a, repo, cwd=tmp_path)
    run("emu", "pack", "-q", "-o", b, repo, cwd=tmp_path)
    assert digest(a) == digest(b)
    out_a, out_b = str(tmp_path / "out_a"), str(tmp_path / "out_b")
    run("emu", "unpack", "-o", out_a, a, cwd=tmp_path)          # each side restores the other's archive
    run("cpu", "unpack", "--cpu", "-o", out_b, b, cwd=tmp_path)
    same_tree(repo, out_a)
    same_tree(repo, out_b)


@pytest.mark.skipif(not (_have_reference() and _have_oracle()), reason="needs the reference package (baseline/_ref or "
                    "$SEEDPACK_REFERENCE) and oracle/_ref")
def test_row_planner_twin_gives_the_reference_archive(tmp_path):
    """a Q8_0 file without a base goes through M21, whose phase C plans the token embedding's rows: the binding's twin of
    that planner (refbind/plan.py, here on CPU tensors) must lead to the archive the reference's own planner leads to"""
    from oracle import ref
    from seedpack_b200 import synthrepo
    repo = str(tmp_path / "repo")
    made = synthrepo.make_repo(repo, "c1-nano", lambda ty, bits, w: ref.quantize(ty, ref.bf16_to_f32(bits), w), seed=3, only=["Q8_0"])
    for p in made["base"]:
        os.remove(p)
    a, b = str(tmp_path / "cpu.seedpack"), str(tmp_path / "emu.seedpack")
    run("cpu", "pack", "--cpu", "-q", "-o", a, repo, cwd=tmp_path)
    r = run("emu", "pack", "-q", "-o", b, repo, cwd=tmp_path)
    assert digest(a) == digest(b)
    out = str(tmp_path / "out")
    run("emu", "unpack", "-o", out, a, cwd=tmp_path)
    same_tree(repo, out)


def test_array_module_residency_and_views():
    """cupy_shim.ndarray on the host side only (no device is touched while nothing asks for one)"""
    from seedpack_b200.refbind import cupy_shim as cp
    a = cp.asarray(np.arange(24, dtype=np.int32).reshape(4, 6))
    assert a.shape == (4, 6) and a.nbytes == 96 and len(a) == 4
    v = a[1:3]
    assert v.shape == (2, 6) and v.get().tolist() == np.arange(6, 18).reshape(2, 6).tolist()
    v[...] = 0                                                   # writes through to the parent
    assert a.get()[1:3].sum() == 0 and int(a[3, 5]) == 23
    u = a.view(np.uint8)
    assert u.shape == (4, 24) and a.reshape(-1).view(np.int64).shape == (12,)
    s = (a + 1).sum(1)
    assert isinstance(s, cp.ndarray) and s.get().tolist() == [21, 6, 6, 129]
    assert bool((a >= 0).all()) and int(cp.cumsum(a.reshape(-1))[-1]) == int(a.get().sum())
    r = cp.full(5, -1, cp.int32)
    r[cp.asarray(np.array([3, 1]))] = cp.arange(2, dtype=cp.int32)
    assert r.get().tolist() == [-1, 1, -1, 0, -1]
    k = cp.asarray(np.array([2, 2, 1, 1, 1, 0], np.int64))
    assert cp.argsort(-k).get().tolist() == [0, 1, 2, 3, 4, 5]    # stable, as CuPy's sorts are
    z = cp.zeros((2, 3), np.uint16)
    z[:, 1:] = cp.asarray(np.ones((2, 2), np.uint16))
    assert z.get().tolist() == [[0, 1, 1], [0, 1, 1]]
    with pytest.raises(NotImplementedError):
        cp.RawModule(code="").get_function("some_kernel_of_the_reference")
    # the integer switches a module's source is compiled with travel to the bindings (M21: SIGN, RANK, SEGA ...)
    m = cp.RawModule(code="#define PB 12\n#define SEGA 4096   // blocks a segment\n#define SIGN 1\n#define TWICE (2 * PB)\nextern \"C\" {}\n")
    assert m.defines == {"PB": 12, "SEGA": 4096, "SIGN": 1}
    from seedpack_b200.refbind import kernels
    assert kernels._m21_flags({"SIGN": 1, "HICF": 1, "RANK": 0}) == 5 and kernels._m21_flags({"PREDA": 1, "RANK": 1}) == 10
    assert cp.uint8 is np.uint8 and isinstance(a, cp.ndarray)
