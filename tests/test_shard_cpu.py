"""The multi-GPU path on CPU: two gloo ranks shard a coding batch by segment, sum their histogram counts through
the host and gather their coded segments; the result must be the bytes a single rank produces (the CPU checker
stands in for the device coder here - the sharding logic is what is under test)."""
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

WORKER = r'''
import os, sys, pickle
sys.path.insert(0, sys.argv[1])
import numpy as np, torch.distributed as dist
from seedpack_b200 import shard
from seedpack_b200.rans import normalize
from oracle import rans as orans
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=int(sys.argv[4]))
rank, world = dist.get_rank(), dist.get_world_size()
rng = np.random.default_rng(3)
SEG, BL, NTAB, n = 1024, 32, 5, 1024 * 11 + 96
bt = rng.integers(0, NTAB, n // BL).astype(np.uint16)
sym = np.where(rng.random(n) < 0.9, 0, rng.integers(0, 64, n)).astype(np.uint8)
nseg = (n + SEG - 1) // SEG
s0, s1 = shard.segment_range(nseg, rank, world)
a, b = s0 * SEG, min(n, s1 * SEG)
counts = np.bincount(np.repeat(bt[a // BL:b // BL], BL).astype(np.int64) * 256 + sym[a:b], minlength=NTAB * 256)
total = shard.sum_counts(counts).reshape(NTAB, 256)
freq, used = normalize(total)
full = np.zeros((NTAB, 256), np.uint16); full[used] = freq
stream, off = orans.encode(sym[a:b], bt[a // BL:b // BL], BL, SEG, full)
lens, data = shard.gather_segments(np.diff(off).astype(np.uint32), stream.tobytes())
if rank == 0:
    pickle.dump({"lens": lens, "stream": data, "freq": freq, "used": used, "sym": sym, "bt": bt}, open(sys.argv[5], "wb"))
dist.destroy_process_group()
'''


def test_two_ranks_give_single_rank_bytes(tmp_path):
    import pickle
    from oracle import rans as orans
    from seedpack_b200.rans import normalize
    port = 29500 + os.getpid() % 2000
    out = str(tmp_path / "r0.pkl")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r), "2", out]) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = pickle.load(open(out, "rb"))
    sym, bt = got["sym"], got["bt"]
    counts = np.bincount(np.repeat(bt, 32).astype(np.int64) * 256 + sym, minlength=5 * 256).reshape(5, 256)
    freq, used = normalize(counts)
    assert np.array_equal(freq, got["freq"]) and np.array_equal(used, got["used"])
    full = np.zeros((5, 256), np.uint16); full[used] = freq
    stream, off = orans.encode(sym, bt, 32, 1024, full)
    assert np.array_equal(np.diff(off).astype(np.uint32), got["lens"]) and stream.tobytes() == got["stream"]


def test_assignment_is_balanced_and_deterministic():
    from seedpack_b200 import shard
    sizes = [100, 90, 80, 10, 10, 10, 5, 5]
    own = shard.assign(sizes, 4)
    load = [sum(s for s, o in zip(sizes, own) if o == r) for r in range(4)]
    assert own == shard.assign(sizes, 4) and max(load) == 100 and min(load) >= 40
    assert shard.assign([], 8) == [] and set(shard.assign([1] * 3, 8)) == {0, 1, 2}
    blocks = shard.row_blocks(4096, 24576, 8)
    assert sum(n for _, n in blocks) == 4096 and len(blocks) == 8 and blocks[0] == (0, 512)
    assert shard.row_blocks(10, 100, 8) == [(0, 10)]
    assert [shard.segment_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
