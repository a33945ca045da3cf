"""Golden digests of whole archives, made with the reference itself (no GPU involved).

For each seeded synthetic repository below: the repository's files are written by seedpack_b200.synthrepo with the
reference's own C quantisers (oracle/_ref), the reference's command line packs it with its `--cpu` path
(tests/tools/refcli.py cpu: the reference package from $SEEDPACK_REFERENCE or baseline/_ref, SOURCE_DATE_EPOCH
fixed), and the SHA-256 of every input file and of the archive go to tests/golden/archive_digests.json.
tests/test_archive_gpu.py must reproduce both on the GPU: the files with the CUDA quantisers, the archive through
seedpack_b200.refbind.

    python tests/golden/make_archive_digests.py [config ...]
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
OUT = os.path.join(HERE, "archive_digests.json")
# "@m28": packed with --method m28 (M24 base codec); "~nobase@m30": the BF16 file removed, packed with --method m30 (sibling quants);
# "~q8only": the Q8_0 file alone, no BF16 file (the M21 codec of Q8_0 blocks: seed.py, gpu2.py, gpu3.py)
CONFIGS = ["c1-nano", "c1-mini", "c4-mini", "c5-mini", "fit-mini", "c1-nano@m28", "sib-mini~nobase@m30", "c1-nano~q8only", "sib-mini~q8only",
           # no BF16 file, default method: the Q8_0 file becomes the seed (seed.py).  The larger case has no disturbed blocks: a
           # flipped byte that makes a Q8_0 scale infinite or NaN puts non-finite weights into the seed, and quantising those
           # runs through float -> int conversions that C leaves undefined (x86 and the GPU give different bytes)
           "c1-nano~nobase", "sib-mini~nobase"]
SEED = 1


def digest(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for b in iter(lambda: f.read(1 << 22), b""):
            h.update(b)
    return h.hexdigest()


def main(configs):
    from oracle import ref
    from seedpack_b200 import synthrepo
    gold = json.load(open(OUT)) if os.path.exists(OUT) else {}
    for cfg in configs:
        with tempfile.TemporaryDirectory() as tmp:
            repo = os.path.join(tmp, "repo")
            t0 = time.time()
            name, _, method = cfg.partition("@")
            name, _, variant = name.partition("~")
            made = synthrepo.make_repo(repo, name, lambda ty, bits, w: ref.quantize(ty, ref.bf16_to_f32(bits), w), seed=SEED,
                                       only=["Q8_0"] if variant == "q8only" else None)
            if variant in ("nobase", "q8only"):
                for p in made["base"]:
                    os.remove(p)
            t1 = time.time()
            arc = os.path.join(tmp, "a.seedpack")
            env = dict(os.environ, SOURCE_DATE_EPOCH="1700000000")
            r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "tools", "refcli.py"), "cpu", "pack", "--cpu", "-q", "-o", arc, repo]
                               + (["--method", method] if method else []),
                               cwd=tmp, env=env, capture_output=True, text=True)
            if r.returncode:
                sys.exit(r.stdout + r.stderr)
            t2 = time.time()
            gold[cfg] = {"seed": SEED, "files": {n: [os.path.getsize(os.path.join(repo, n)), digest(os.path.join(repo, n))]
                                                 for n in sorted(os.listdir(repo))},
                         "archive": [os.path.getsize(arc), digest(arc)]}
            print(f"{cfg}: repository {t1 - t0:.0f} s, reference --cpu pack {t2 - t1:.0f} s, archive {os.path.getsize(arc)} B", flush=True)
        with open(OUT, "w") as f:
            json.dump(gold, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main(sys.argv[1:] or CONFIGS)
