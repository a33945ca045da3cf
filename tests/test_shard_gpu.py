"""The sharded path on two GPUs: one process per GPU, a coding batch cut by segment range, each rank quantising the
rows behind its segments, counts added through the host (gloo), tables normalised on every rank alike, coded segments
gathered in order on rank 0.  The gathered batch must be the bytes one GPU produces for the whole batch."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

WORKER = r'''
import os, sys, pickle
sys.path.insert(0, sys.argv[1])
import numpy as np, torch, torch.distributed as dist
from seedpack_b200 import shard
from seedpack_b200.shardcode import sharded_batch, make_case
rank, world = int(sys.argv[3]), int(sys.argv[4])
torch.cuda.set_device(rank % torch.cuda.device_count())
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=rank, world_size=world)
out = {}
for T in (12, 17, 8):
    case = make_case(T, [(512, 5120), (128, 17408)], seed=5)
    buf = sharded_batch(T, case, rank, world)
    if rank == 0:
        out[T] = buf
if rank == 0:
    pickle.dump(out, open(sys.argv[5], "wb"))
dist.destroy_process_group()
'''


def _run(world, tmp_path, tag):
    port = 29500 + (os.getpid() + world * 7) % 2000
    out = str(tmp_path / f"r0_{tag}.pkl")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r), str(world), out]) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    import pickle
    return pickle.load(open(out, "rb"))


def test_two_gpus_give_the_single_gpu_batch(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    one = _run(1, tmp_path, "one")
    two = _run(2, tmp_path, "two")
    assert one.keys() == two.keys()
    for T in one:
        assert one[T] == two[T], f"type {T}: the batch depends on the number of GPUs"


def test_ranks_on_one_gpu_give_the_single_rank_batch(tmp_path):
    """the same with both ranks on one GPU (their kernels do not wait on one another: plain launches, the exchange is
    through the host), so that the sharded code path is covered where only one GPU is at hand"""
    one = _run(1, tmp_path, "one")
    three = _run(3, tmp_path, "three")
    for T in one:
        assert one[T] == three[T], f"type {T}: the batch depends on the number of ranks"
