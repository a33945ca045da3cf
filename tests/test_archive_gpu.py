"""Whole archives on the GPU against the reference's own.

The reference's unmodified command line, repository code and container (the `seedpack` package found by
seedpack_b200.refbind: $SEEDPACK_REFERENCE or baseline/_ref) run with every kernel served by libseedgrow.so
(`python -m seedpack_b200.refbind`).  Checked here:

  * golden digests (tests/golden/archive_digests.json, made without a GPU by tests/golden/make_archive_digests.py:
    repository files by the reference's C quantisers, archive by the reference's `--cpu` path): the synthetic
    repositories regenerated with the CUDA quantisers have the same file digests, and the archive packed on the GPU has
    the same digest as the reference's `--cpu` archive - byte-identical archives for the 0.6B-shaped repository without
    importance matrix (three quant files), the 9B-shaped one with 21 importance-matrix quants and the 27B-shaped one
    in two shards with 24 quants and altered tensor types, at reduced sizes; a repository whose legacy quants were
    made with another importance matrix than the published one (the packer fits it back: seedpack/imxfit.py over
    sg_dm_gram and friends); the smallest repository packed with --method m28 (the M24 base codec); and the 0.6B shape at reduced size
    repository WITHOUT its BF16 file packed with --method m30 (seedpack/siblings.py: the quants of a tensor coded in a
    chain, each predicted from the precision-weighted mean of those before it: sg_sib_* and the QR coder's seedless and
    explicit-seed paths);
  * both ways on one box: the reference's `--cpu` run packs the smallest repository here too, the archives are
    compared byte for byte, and each side unpacks the OTHER side's archive to files equal to the originals;
  * `test` / `unpack` on the GPU restore every file of every archive (the reference's own BLAKE3 check plus a
    comparison with the inputs).

In the GPU runs `seedpack.cpukernels.RawModule` raises and the oracle is not imported by the packing process.
"""
import hashlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLD = json.load(open(os.path.join(HERE, "golden", "archive_digests.json")))
pytestmark = pytest.mark.gpu


def digest(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for b in iter(lambda: f.read(1 << 22), b""):
            h.update(b)
    return h.hexdigest()


def gpu_quantizer():
    import torch
    from seedpack_b200.gpuquant import GPUQuant
    gq = GPUQuant(0)

    def q(ty, bits, w):
        x = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().reshape(-1)
        return gq.quantize_tensors(ty, [(x, bits.shape[1])], [w])[0]
    return q


def bound(*args, cwd):
    """the reference's command line on the bound kernels, in a child process"""
    env = dict(os.environ, SOURCE_DATE_EPOCH="1700000000", PYTHONPATH=ROOT)
    env.pop("SEEDPACK_CPU", None)
    r = subprocess.run([sys.executable, "-m", "seedpack_b200.refbind", *args], cwd=cwd, env=env, capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r


def reference_cpu(*args, cwd):
    env = dict(os.environ, SOURCE_DATE_EPOCH="1700000000")
    r = subprocess.run([sys.executable, os.path.join(HERE, "tools", "refcli.py"), "cpu", *args], cwd=cwd, env=env, capture_output=True,
                       text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r


def same_tree(a, b):
    names = sorted(os.listdir(a))
    assert names == sorted(os.listdir(b))
    for n in names:
        assert digest(os.path.join(a, n)) == digest(os.path.join(b, n)), n


def need_reference():
    from seedpack_b200 import refbind
    if not refbind.available():
        pytest.fail("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE): archives cannot be made")


@pytest.mark.parametrize("config", ["c1-nano", "c1-mini", "c4-mini", "c5-mini", "fit-mini", "c1-nano@m28", "sib-mini~nobase@m30",
                                    "c1-nano~q8only", "sib-mini~q8only", "c1-nano~nobase", "sib-mini~nobase"])
def test_archive_equals_the_references(config, tmp_path):
    need_reference()
    from seedpack_b200 import synthrepo
    if config not in GOLD:
        pytest.fail(f"no golden digests for {config}")
    gold = GOLD[config]
    repo = str(tmp_path / "repo")
    name, _, method = config.partition("@")                # "@m28": packed with --method m28 (the M24 base codec)
    name, _, variant = name.partition("~")                 # "~nobase": the BF16 file removed ("@m30": the quants code one another)
    # "~nobase" with no method: the Q8_0 file takes the BF16 file's place as the seed the other files are predicted from (seed.py);
    # "~q8only": the Q8_0 file alone with no BF16 file, which the reference packs with its M21 codec of Q8_0 blocks
    made = synthrepo.make_repo(repo, name, gpu_quantizer(), seed=gold["seed"], only=["Q8_0"] if variant == "q8only" else None)
    if variant in ("nobase", "q8only"):
        for p in made["base"]:
            os.remove(p)
    # the repository itself: every quant file written by the CUDA quantisers equals the one the reference's C code wrote
    assert sorted(os.listdir(repo)) == sorted(gold["files"])
    for n, (size, dg) in gold["files"].items():
        assert os.path.getsize(os.path.join(repo, n)) == size and digest(os.path.join(repo, n)) == dg, n
    arc = str(tmp_path / "gpu.seedpack")
    bound("pack", "-q", "-o", arc, repo, *(["--method", method] if method else []), cwd=tmp_path)
    assert [os.path.getsize(arc), digest(arc)] == gold["archive"]
    bound("test", arc, cwd=tmp_path)
    out = str(tmp_path / "out")
    bound("unpack", "-o", out, arc, cwd=tmp_path)
    same_tree(repo, out)


def test_pack_and_unpack_interoperate_both_ways(tmp_path):
    need_reference()
    from seedpack_b200 import synthrepo
    repo = str(tmp_path / "repo")
    synthrepo.make_repo(repo, "c1-nano", gpu_quantizer(), seed=7)
    a, b = str(tmp_path / "gpu.seedpack"), str(tmp_path / "cpu.seedpack")
    bound("pack", "-q", "-o", a, repo, cwd=tmp_path)
    reference_cpu("pack", "--cpu", "-q", "-o", b, repo, cwd=tmp_path)
    assert digest(a) == digest(b)
    out_a, out_b = str(tmp_path / "from_gpu_archive"), str(tmp_path / "from_cpu_archive")
    reference_cpu("unpack", "--cpu", "-o", out_a, a, cwd=tmp_path)
    bound("unpack", "-o", out_b, b, cwd=tmp_path)
    same_tree(repo, out_a)
    same_tree(repo, out_b)


def test_single_pass_kernel_bindings_give_the_same_archive(tmp_path):
    """qr.encode / qr.decode of the reference left as they are (its qr_hist / qr_enc / qr_dec launches bound one to one,
    the model run twice per block) give the archive the staged coder gives"""
    need_reference()
    from seedpack_b200 import synthrepo
    gold = GOLD["c1-nano"]
    repo = str(tmp_path / "repo")
    synthrepo.make_repo(repo, "c1-nano", gpu_quantizer(), seed=gold["seed"])
    arc = str(tmp_path / "gpu.seedpack")
    env = dict(os.environ, SOURCE_DATE_EPOCH="1700000000", PYTHONPATH=ROOT, SEEDGROW_QR_SINGLE_PASS="1")
    r = subprocess.run([sys.executable, "-m", "seedpack_b200.refbind", "pack", "-q", "-o", arc, repo], cwd=tmp_path, env=env,
                       capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert [os.path.getsize(arc), digest(arc)] == gold["archive"]
    r = subprocess.run([sys.executable, "-m", "seedpack_b200.refbind", "test", arc], cwd=tmp_path, env=env, capture_output=True, text=True,
                       timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def test_disturbed_seed_round_trips(tmp_path):
    """a repository without its BF16 file whose Q8_0 seed has disturbed blocks (some scales infinite or NaN, so the weights
    the other files are re-quantised from are not finite): the archive is not compared with x86's - C leaves the float ->
    int conversions of such values undefined - but packing, testing and unpacking on the GPU give the files back"""
    need_reference()
    from seedpack_b200 import synthrepo
    repo = str(tmp_path / "repo")
    made = synthrepo.make_repo(repo, "c1-mini", gpu_quantizer(), seed=1)
    for p in made["base"]:
        os.remove(p)
    arc = str(tmp_path / "gpu.seedpack")
    bound("pack", "-q", "-o", arc, repo, cwd=tmp_path)
    bound("test", arc, cwd=tmp_path)
    out = str(tmp_path / "out")
    bound("unpack", "-o", out, arc, cwd=tmp_path)
    same_tree(repo, out)
