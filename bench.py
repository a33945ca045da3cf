#!/usr/bin/env python
"""Benchmarks of the re-quantise / residual / rANS path.

Default workload `pack`: a seeded synthetic model repository of the 0.6B shape (28 layers, hidden 1024, FFN 3072,
vocabulary 151936; BF16 base + Q8_0, Q4_K_M-shaped and Q6_K files with 0.5 % of the blocks disturbed) is packed into an
archive and the archive is tested (every file restored in memory and checked) - the reference's own command line,
repository code and container running on this library's kernels (seedpack_b200.refbind).  A step = one pack + one
test.  Metric: GB/s of GGUF bytes, pack and unpack.

    e2e      wall clock through the command-line entry points: files read from disk, host <-> device copies, zstd,
             hashing, container writes included
    value    the same bytes over the device time of the step's library calls (CUDA events around every C-ABI call):
             what the kernels alone sustain, with the host pipeline taken out

    python bench.py --gpus N --steps K --warmup W          (this repo's CUDA path)
    python bench.py --impl reference ...                   (the reference's own --cpu path on the host cores, on a
                                                            bounded sample: one layer of the same shape)
    python bench.py --workload quant | rans | qr | r2      (kernel-level workloads: the quantiser sweep over one
                                                            4096 x 12288 tensor and 25 types; the coders)

Multi-GPU (`pack`): every rank packs and tests a repository of its own (seed 1 + rank) on its GPU - weak scaling, the
maximum over the ranks' times; no collective on the data path.  `--workload shard` cuts ONE window of tensors over the
ranks by rANS segment (strong scaling; the digest of the coded batches does not depend on N).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NROWS, NPR = 4096, 12288          # --rows overrides NROWS for small profiling captures
QFUN = {2: ("q4_0", 32, 18), 3: ("q4_1", 32, 20), 6: ("q5_0", 32, 22), 7: ("q5_1", 32, 24),
        8: ("q8_0", 32, 34), 10: ("q2_K", 256, 84), 11: ("q3_K", 256, 110), 12: ("q4_K", 256, 144),
        13: ("q5_K", 256, 176), 14: ("q6_K", 256, 210), 16: ("iq2_xxs", 256, 66), 17: ("iq2_xs", 256, 74),
        18: ("iq3_xxs", 256, 98), 19: ("iq1_s", 256, 50), 20: ("iq4_nl", 32, 18), 21: ("iq3_s", 256, 110),
        22: ("iq2_s", 256, 82), 23: ("iq4_xs", 256, 136), 29: ("iq1_m", 256, 56), 42: ("q2_0", 64, 18),
        34: ("tq1_0", 256, 54), 35: ("tq2_0", 256, 66), 39: ("mxfp4", 32, 17), 40: ("nvfp4", 64, 36), 41: ("q1_0", 128, 18)}
NO_IMX_TOO = [2, 3, 6, 7, 10, 11, 12, 13, 14, 18, 20, 21, 22, 23, 29]     # types whose matrix-free routine differs
NO_IMX_ONLY = [34, 35, 39, 40, 41]                                        # types that take no importance matrix
CASES = [(t, True) for t in sorted(QFUN) if t not in NO_IMX_ONLY] + [(t, False) for t in NO_IMX_TOO + NO_IMX_ONLY]


# fp32 add / mul thread instructions and all thread instructions per weight of every launch of the sweep, counted by ncu
# on a 256-row tensor (profiles/quant_fp32_ops_ncu.md gives the command); the counts per weight do not depend on the
# number of rows.  Launches with fewer than 30 fp32 operations per weight are bound by memory traffic and instruction
# issue for the packing; the others by the quantisers' scale searches: fp32 add / mul issue.
OPS = {"q6_K+imx": [186.2, 286.2], "iq2_xxs+imx": [695.1, 2780.0], "iq2_xs+imx": [1118.8, 5405.5], "iq3_xxs+imx": [1795.9, 4190.8],
       "iq1_s+imx": [576.5, 1235.0], "iq4_nl+imx": [143.6, 646.4], "iq3_s+imx": [1287.9, 2870.3], "iq2_s+imx": [467.9, 1669.1],
       "iq4_xs+imx": [144.3, 650.9], "iq1_m+imx": [379.4, 1044.6], "q2_0+imx": [2.1, 13.7], "q4_0": [2.3, 17.0], "q4_1": [3.5, 20.0],
       "q5_0": [2.3, 20.1], "q5_1": [3.5, 20.2], "q2_K": [286.8, 445.3], "q3_K": [28.3, 115.1], "q4_K": [356.9, 522.5],
       "q5_K": [277.5, 419.6], "q6_K": [186.9, 285.7], "iq3_xxs": [1800.5, 4204.2], "iq4_nl": [140.6, 637.8], "iq3_s": [1281.3, 2860.3],
       "iq2_s": [461.6, 1652.5], "iq4_xs": [145.5, 643.5], "iq1_m": [368.9, 996.0], "tq1_0": [2.3, 25.7], "tq2_0": [2.3, 22.7],
       "mxfp4": [0.6, 33.8], "nvfp4": [1.1, 33.2], "q1_0": [1.0, 17.8], "q4_0+imx": [181.5, 251.4], "q4_1+imx": [646.9, 829.2],
       "q5_0+imx": [181.4, 253.8], "q5_1+imx": [646.9, 831.7], "q8_0+imx": [2.4, 16.2], "q2_K+imx": [873.5, 1267.1],
       "q3_K+imx": [346.6, 547.8], "q4_K+imx": [702.4, 940.8], "q5_K+imx": [702.3, 947.7]}
SMS, FP32_LANES, ISSUE_SLOTS = 148, 128, 4


def bound_of(name):
    return "hbm" if OPS[name][0] < 30 else "fp32_issue"


# DRAM traffic of one full-size launch (bytes read + written), from ncu captures on 1024 of the 4096 rows scaled by 4
# (the traffic grows with the rows; profiles/quant_lattice_queue_ncu_full.md).  Writes that were still in L2 when the
# captured kernel ended are not in the counter.
NCU_TRAFFIC = {"iq2_xs+imx": 4 * 25.843456e6, "iq2_xxs+imx": 4 * 25.738752e6}


def quant_bytes(t, nrows=None, npr=NPR):
    _, qk, bs = QFUN[t]
    return (NROWS if nrows is None else nrows) * npr // qk * bs


def algo_bytes(t, imx, nrows=None, npr=NPR):
    """algorithmic bytes of one launch: BF16 in + blocks out + importance matrix"""
    nrows = NROWS if nrows is None else nrows
    return 2 * nrows * npr + quant_bytes(t, nrows, npr) + (4 * npr if imx else 0)


def workload_text():
    n_imx = sum(1 for _, use in CASES if use)
    return (f"quantizer sweep, BF16 {NROWS}x{NPR} + imatrix {NPR}, {len(CASES)} launches per step "
            f"({n_imx} with imatrix, {len(CASES) - n_imx} without)")


_SYNTH = {}


def synth_tensor(seed):
    """(bf16 bits [NROWS, NPR], importance matrix [NPR]) of the benchmark tensor, cached per seed"""
    from tests import synth
    if seed not in _SYNTH:
        _SYNTH[seed] = (synth.weights(NROWS, NPR, seed, edge_cases=False), synth.imatrix(NPR, seed))
    return _SYNTH[seed]


def default_ref_rows(threads):
    """rows of the tensor the CPU baseline quantises per step: about a second of wall time on all cores"""
    return int(min(NROWS, max(64, 8 * threads)))


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """nvidia-smi clocks and throttle reasons while the timed region runs"""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                o = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True, timeout=5).stdout.strip()
                if o:
                    self.rows.append([c.strip() for c in o.split(",")])
            except Exception:
                pass
            time.sleep(0.2)

    def summary(self):
        self.stop_flag = True
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(len(r) > 2 + k and r[2 + k] == "Active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


# ------------------------------------------------------------------------------------------------------
def cpu_reference_run(rows, threads, seed=1, cases=CASES):
    """the reference's C quantisers (oracle/_ref) on `rows` rows of the benchmark tensor, every case once.
    Returns (seconds, quant bytes produced, per-case seconds)."""
    from oracle import ref
    from tests import synth
    bits, imx = synth_tensor(seed)
    x = synth.bf16_bits_to_f32(bits[:rows]).reshape(rows, NPR)
    for t in {t for t, _ in cases}:
        ref._init(t, 0)            # table construction is set-up, not the timed path
    per, total_b = {}, 0
    t_all = time.perf_counter()
    for t, use in cases:
        t0 = time.perf_counter()
        ref.quantize(t, x, imx if use else None, threads=threads)
        per[f"{QFUN[t][0]}{'+imx' if use else ''}"] = time.perf_counter() - t0
        total_b += quant_bytes(t, rows)
    return time.perf_counter() - t_all, total_b, per


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref
    threads = os.cpu_count() or 1
    rows = args.ref_rows or default_ref_rows(threads)
    cfg = {"workload": workload_text() + ", one tensor per GPU", "l2": "flushed between launches (256 MiB memset inside the timed region)"}
    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libggmlq_ref.so not built (needs the reference tree at build time)"}))
        return
    for _ in range(args.warmup):
        cpu_reference_run(min(rows, 8), threads)
    times, nbytes = [], 0
    for _ in range(args.steps):
        dt, nbytes, _ = cpu_reference_run(rows, threads)
        times.append(dt)
    tot = sum(times)
    val = nbytes * len(times) / tot / 1e9
    line = {"impl": "reference", "metric": "quantizer sweep GB/s of GGUF bytes regrown", "value": val, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot / len(times) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": cfg,
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "reference",
                             "sample": f"first {rows} of {NROWS} rows of the same tensor ({100 * rows / NROWS:.1f}% of it), all {len(CASES)} launches per step"},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from seedpack_b200.gpuquant import GPUQuant

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    gq = GPUQuant(local)

    bits, imx = synth_tensor(1 + rank)
    hx = torch.from_numpy(bits.view(np.int16)).pin_memory()
    himx = torch.from_numpy(imx).pin_memory()
    x = hx.to(dev).view(torch.bfloat16).reshape(-1)
    w = himx.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out_bytes = sum(quant_bytes(t) for t, _ in CASES)

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in CASES]

    def step(record=False):
        launches = 0
        for k, (t, use) in enumerate(CASES):
            flush.zero_()                                   # evict the tensor from L2 between launches
            if record:
                ev[k][0].record()
            gq.quantize_tensors(t, [(x, NPR)], [w if use else None], device=True)
            if record:
                ev[k][1].record()
            launches += 2 if (use and t in (2, 3, 6, 7)) else 1
        return launches

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    per = np.zeros(len(CASES))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    e0.record()
    for _ in range(args.steps):
        launches += step(record=True)
        torch.cuda.synchronize()                            # per-launch events are read between steps
        per += np.array([a.elapsed_time(b) for a, b in ev])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.summary()

    # end to end through the public API: host BF16 + importance matrix in, quantised bytes out to the host.  The copies
    # back run on a second stream behind each launch, so they overlap the next launch (every case has its own range
    # of the pinned output buffer)
    hall = torch.empty(out_bytes + 64 * len(CASES), dtype=torch.uint8).pin_memory()
    copy_stream = torch.cuda.Stream(dev)

    def e2e_step():
        xd = hx.to(dev, non_blocking=True).view(torch.bfloat16).reshape(-1)
        wd = himx.to(dev, non_blocking=True)
        pos, keep = 0, []
        for t, use in CASES:
            y = gq.quantize_tensors(t, [(xd, NPR)], [wd if use else None], device=True)[0]
            done = torch.cuda.Event()
            done.record()
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(done)
                hall[pos:pos + y.numel()].copy_(y, non_blocking=True)
            y.record_stream(copy_stream)
            keep.append(y)
            pos += y.numel() + 64
        copy_stream.synchronize()
        torch.cuda.synchronize()

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_n = max(1, min(args.steps, 3))
    for _ in range(e2e_n):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_n

    if world > 1:
        tms = torch.tensor([ms, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(tms[0]), float(tms[1])
    ms_step = ms / args.steps
    value = world * out_bytes / (ms_step * 1e-3) / 1e9

    line = None
    if rank == 0:
        peak, peak_kind = peaks()
        per_ms = per / args.steps
        table = {}
        clk = (clocks.get("sm_mhz") or 1965.0) * 1e6
        fp32_peak = SMS * FP32_LANES * clk / 1e12               # T fp32 add / mul per second at the sampled clock
        nw = NROWS * NPR
        for k, (t, use) in enumerate(CASES):
            name = case_name(t, use)
            sec = per_ms[k] * 1e-3
            a = algo_bytes(t, use) / sec / 1e9
            row = {"ms": round(float(per_ms[k]), 4), "bound": bound_of(name), "algo_gbs": round(a, 1),
                   "gguf_gbs": round(quant_bytes(t) / sec / 1e9, 2), "hbm_frac": round(a / peak, 4),
                   "issue_slots_busy": round(OPS[name][1] * nw / 32 / sec / (SMS * ISSUE_SLOTS * clk), 3)}
            if row["bound"] == "fp32_issue":
                row["fp32_tops"] = round(OPS[name][0] * nw / sec / 1e12, 2)
                row["fp32_frac"] = round(OPS[name][0] * nw / sec / 1e12 / fp32_peak, 3)
            table[name] = row
        dom = int(np.argmax(per_ms))
        dt, duse = CASES[dom]
        dname = case_name(dt, duse)
        ach = algo_bytes(dt, duse) / (per_ms[dom] * 1e-3) / 1e9
        # CPU baseline: the reference's C code on a bounded row sample, all host threads
        cpu = None
        try:
            from oracle import ref
            if ref.available():
                threads = os.cpu_count() or 1
                rows = args.ref_rows or default_ref_rows(threads)
                dtc, nb, _ = cpu_reference_run(rows, threads)
                cpu = {"value": nb / dtc / 1e9, "unit": "GB/s", "cores": threads, "kind": "reference",
                       "sample": f"first {rows} of {NROWS} rows of the same tensor, all {len(CASES)} launches once"}
        except Exception as e:                                   # the baseline is reported, never required
            cpu = {"value": None, "unit": "GB/s", "cores": 0, "kind": "reference", "sample": f"failed: {e}"}
        line = {"metric": "quantizer sweep GB/s of GGUF bytes regrown", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload_text() + ", one tensor per GPU",
                           "l2": "flushed between launches (256 MiB memset inside the timed region)"},
                "per_type": table,
                "clocks": clocks,
                "e2e": {"value": world * out_bytes / e2e_s / 1e9, "unit": "GB/s",
                        "h2d_bytes_per_step": int(world * (hx.numel() * 2 + himx.numel() * 4)), "d2h_bytes_per_step": int(world * out_bytes)},
                "gpu_launches": int(launches),
                "roofline": quant_roofline(dname, table[dname], ach, peak, peak_kind, fp32_peak),
                "cpu_baseline": cpu}
    if world > 1 and not getattr(args, "keep_group", False):
        dist.destroy_process_group()
    return line


# ------------------------------------------------------------------------------------------------------
# `pack`: the reference's command line (pack, test) on a synthetic repository, kernels from this library
def _bench_tmp():
    """where the benchmark's repository and archive live: $SEEDGROW_BENCH_TMP, else RAM-backed /dev/shm when it has
    room (inputs as hot as a page cache would hold them), else the system's temporary directory"""
    import shutil
    import tempfile
    d = os.environ.get("SEEDGROW_BENCH_TMP")
    if not d:
        try:
            world = int(os.environ.get("WORLD_SIZE", "1"))          # every rank keeps a repository, its archive and an unpacked copy
            d = "/dev/shm" if shutil.disk_usage("/dev/shm").free > (8 << 30) * world + (4 << 30) else None
        except OSError:
            d = None
    return tempfile.mkdtemp(prefix="seedgrow-bench-", dir=d)


def _repo_text(cfg_name):
    from seedpack_b200 import synthrepo
    c = synthrepo.CONFIGS[cfg_name]
    return (f"synthetic repository '{cfg_name}': {c['layers']} layers, hidden {c['hidden']}, FFN {c['ffn']}, vocabulary {c['vocab']}, "
            f"BF16 base in {c['shards']} file(s) + {len(synthrepo.file_labels(c))} quant files"
            f"{' made with an importance matrix' if c['imatrix'] else ', no importance matrix'}, {100 * c['flip']:.1f}% of blocks disturbed")


def _file_digest(path):
    import hashlib
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for b in iter(lambda: f.read(1 << 22), b""):
            h.update(b)
    return h.hexdigest()


def _quiet(fn, *a):
    """run a command-line entry point with its progress output discarded; SystemExit with a message is an error"""
    import contextlib
    import io
    buf = io.StringIO()
    try:
        with contextlib.redirect_stdout(buf):
            fn(*a)
    except SystemExit as e:
        if e.code not in (None, 0):
            raise RuntimeError(f"{a}: {e.code}\n{buf.getvalue()[-2000:]}")
    return buf.getvalue()


def _reference_cli():
    """the reference's command-line module with its own CPU kernels (SEEDPACK_CPU=1), for the CPU legs"""
    from seedpack_b200 import refbind
    ref = refbind.find_reference()
    if ref is None:
        return None
    import importlib.util
    os.environ["SEEDPACK_CPU"] = "1"
    os.environ.setdefault("SEEDPACK_CACHE", os.path.join(ROOT, "oracle", "_build", "refcache"))
    os.environ.setdefault("NUMBA_CACHE_DIR", os.path.join(ROOT, "oracle", "_build", "numba"))
    os.makedirs(os.environ["SEEDPACK_CACHE"], exist_ok=True)
    if ref not in sys.path:
        sys.path.insert(0, ref)
    if importlib.util.find_spec("zstandard") is None:
        from seedpack_b200 import zstd
        sys.modules["zstandard"] = zstd
    from seedpack import cli
    return cli


PACK_METRIC = "pack/unpack GB/s of GGUF bytes"


def pack_config(repo, gpus, without_base="no"):
    """the `config` object of the pack workload, the same in this library's line and in the reference arm's"""
    less = {"no": "", "all": "; the BF16 file removed before packing (the Q8_0 file is the seed)",
            "q8": "; the Q8_0 file alone, no BF16 file (M21)"}[without_base]
    return {"workload": _repo_text(repo) + less + (", one repository per GPU" if gpus > 1 else ""),
            "step": "pack + test of the repository; bytes per step = 2 x repository bytes",
            "l2": "inputs larger than L2 (base 1.2 GB, files 1.5 GB)"}
SAMPLE = "c1-micro"


def run_reference_pack(args):
    """--impl reference: the reference's own `pack --cpu` and `test --cpu` on the host cores, on a bounded sample of the
    workload (one layer of the same shape), in this process"""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import shutil
    threads = os.cpu_count() or 1
    cfg = pack_config(args.repo, args.gpus)
    cli = _reference_cli()
    if cli is None:
        print(json.dumps({"impl": "reference", "unavailable": "the reference package is not installed under baseline/_ref (nor $SEEDPACK_REFERENCE)"}))
        return
    tmp = _bench_tmp()
    try:
        repo = args.repo_dir
        if not repo:
            from oracle import ref as oref
            from seedpack_b200 import synthrepo
            repo = os.path.join(tmp, "repo")
            synthrepo.make_repo(repo, SAMPLE, lambda ty, bits, w: oref.quantize(ty, oref.bf16_to_f32(bits), w), seed=1, keep_weights=True)
        nbytes = sum(os.path.getsize(os.path.join(repo, n)) for n in os.listdir(repo))
        arc = os.path.join(tmp, "ref.seedpack")
        tp = tu = 0.0
        warm = min(args.warmup, 1)
        for k in range(warm + args.steps):
            t0 = time.perf_counter()
            _quiet(cli.main, ["pack", "--cpu", "-q", "-f", "-o", arc, repo])
            t1 = time.perf_counter()
            _quiet(cli.main, ["test", "--cpu", arc])
            t2 = time.perf_counter()
            if k >= warm:
                tp += t1 - t0; tu += t2 - t1
        val = 2 * nbytes * args.steps / (tp + tu) / 1e9
        sample = (f"'{SAMPLE}' (one layer of the 0.6B shape, vocabulary 4096: {nbytes} bytes, {100 * nbytes / 2.7e9:.1f}% of the full repository), "
                  f"python -m seedpack pack --cpu + test --cpu, {threads} host threads")
        line = {"impl": "reference", "metric": PACK_METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": warm, "ms_per_step": (tp + tu) / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
                "pack_gbs": nbytes * args.steps / tp / 1e9, "unpack_gbs": nbytes * args.steps / tu / 1e9,
                "archive_sha256": _file_digest(arc),
                "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "reference", "sample": sample},
                "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def run_pack(args):
    import shutil
    import torch
    import torch.distributed as dist
    from seedpack_b200 import _lib, refbind, synthrepo
    from seedpack_b200.gpuquant import GPUQuant
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    if not refbind.available():
        raise RuntimeError("the reference package is not here (baseline/_ref or $SEEDPACK_REFERENCE): pack needs its host code")
    gq = GPUQuant(local)

    def quantize(ty, bits, w):
        x = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev).reshape(-1)
        return gq.quantize_tensors(ty, [(x, bits.shape[1])], [w])[0]

    tmp = _bench_tmp()
    try:
        os.environ.setdefault("SOURCE_DATE_EPOCH", "1700000000")
        repo = os.path.join(tmp, "repo")
        made = synthrepo.make_repo(repo, args.repo, quantize, seed=1 + rank, keep_weights=args.without_base == "no",
                                   only=["Q8_0"] if args.without_base == "q8" else None)
        nbytes = made["bytes"]
        base_bytes = sum(os.path.getsize(p) for p in made["base"])
        if args.without_base != "no":               # the Q8_0 file becomes the seed: M21 codes it, the others follow from it
            for p in made["base"]:
                os.remove(p)
            nbytes = sum(os.path.getsize(os.path.join(repo, n)) for n in os.listdir(repo))
        arc = os.path.join(tmp, "a.seedpack")
        refbind.install()
        from seedpack import cli
        from seedpack_b200.refbind import cupy_shim

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def step():
            t0 = time.perf_counter()
            _quiet(cli.main, ["pack", "-q", "-f", "-o", arc, repo])
            t1 = time.perf_counter()
            _quiet(cli.main, ["test", arc])
            return t1 - t0, time.perf_counter() - t1

        for _ in range(args.warmup):
            step()
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        cupy_shim.STATS.update(h2d=0, d2h=0)
        _lib.COPIES.update(h2d=0, d2h=0)
        _lib.timing_start(calls=True)
        tp = tu = 0.0
        t_all = time.perf_counter()
        for _ in range(args.steps):
            a, b = step()
            tp += a; tu += b
        barrier()
        wall = time.perf_counter() - t_all
        calls = _lib.timing_stop(counts=True)
        clocks = sampler.summary()
        dev_ms = sum(v[0] for v in calls.values())
        h2d = (cupy_shim.STATS["h2d"] + _lib.COPIES["h2d"]) / args.steps
        d2h = (cupy_shim.STATS["d2h"] + _lib.COPIES["d2h"]) / args.steps
        # every file back, compared with what went in
        out = os.path.join(tmp, "out")
        _quiet(cli.main, ["unpack", "-o", out, arc])
        names = sorted(os.listdir(repo))
        exact = sum(1 for n in names if os.path.exists(os.path.join(out, n)) and _file_digest(os.path.join(out, n)) == _file_digest(os.path.join(repo, n)))
        shutil.rmtree(out, ignore_errors=True)
        if world > 1:
            t = torch.tensor([wall, dev_ms, tp, tu], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            wall, dev_ms, tp, tu = (float(x) for x in t)
            c = torch.tensor([nbytes, exact, len(names), h2d, d2h], device=dev, dtype=torch.float64)
            dist.all_reduce(c, op=dist.ReduceOp.SUM)
            nbytes_all, exact, total, h2d, d2h = float(c[0]), int(c[1]), int(c[2]), float(c[3]), float(c[4])
        else:
            nbytes_all, total = nbytes, len(names)
        if rank == 0:
            peak, peak_kind = peaks()
            per = {k: {"ms": round(v[0] / args.steps, 3), "calls": v[1] // args.steps} for k, v in sorted(calls.items(), key=lambda kv: -kv[1][0])}
            dom = next(iter(per)) if per else None
            line = {"metric": PACK_METRIC, "value": 2 * nbytes_all * args.steps / (dev_ms * 1e-3) / 1e9 if dev_ms else None, "unit": "GB/s",
                    "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
                    "wall_ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                    "dtype": "f32", "data": "synthetic",
                    "config": pack_config(args.repo, world, args.without_base),
                    "value_is": "bytes over the summed device time of the step's library calls (CUDA events around each call); e2e is the wall clock",
                    "repository_bytes": int(nbytes), "library_calls": per,
                    "clocks": clocks,
                    "e2e": {"value": 2 * nbytes_all * args.steps / wall / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(h2d),
                            "d2h_bytes_per_step": int(d2h), "pack_gbs": nbytes_all * args.steps / tp / 1e9,
                            "unpack_gbs": nbytes_all * args.steps / tu / 1e9},
                    "bit_exact_files": f"{exact}/{total}", "archive_sha256": _file_digest(arc),
                    "gpu_launches": int(sum(v[1] for v in calls.values())),
                    "roofline": pack_roofline(per, dom, args, peak, peak_kind, clocks, base_bytes if args.without_base == "no" else 0,
                                              os.path.getsize(arc))}
            line["cpu_baseline"] = pack_cpu_baseline(args, tmp, quantize, cli) if world == 1 and args.without_base == "no" else None
            if world == 1 and not args.no_kernels:
                line["kernels"] = kernel_workloads(args)
            print(json.dumps(line))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
        if world > 1:
            dist.destroy_process_group()


def kernel_workloads(args):
    """the kernel-level workloads, a few steps each, for the default line: the quantiser sweep over one 4096 x 12288 tensor
    (per-type table, fp32-issue roofline of its largest launch) and the three coders, each with its own clock samples"""
    import copy
    out = {}
    a = copy.copy(args)
    a.steps, a.warmup = 3, 3
    try:
        q = run_ours(a)
        out["quant_sweep"] = {k: q[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "per_type", "clocks", "e2e", "roofline")}
    except Exception as e:
        out["quant_sweep"] = {"failed": str(e)}
    a.steps, a.warmup, a.tensors, a.qr_types = 2, 1, 4, "8,12,17"
    for name, fn in (("rans", run_rans), ("qr", run_qr), ("r2", run_r2)):
        try:
            l = fn(a)
            out[name] = {k: l[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "clocks", "e2e", "roofline")}
        except Exception as e:
            out[name] = {"failed": str(e)}
    return out


def pack_roofline(per, dom, args, peak, peak_kind, clocks, base_bytes=0, coded_bytes=0):
    """the library call with the largest share of the step's device time, against the memory roofline: the base codec's
    calls move the BF16 base (statistics: rows, then columns twice; coders: base + coded stream)"""
    if dom is None:
        return None
    algo = {"sg_r2_stats": 3 * base_bytes, "sg_r2_decode": base_bytes + coded_bytes, "sg_r2_encode": base_bytes + coded_bytes,
            "sg_r2_hist": base_bytes, "sg_row_hash": base_bytes}.get(dom)
    ach = algo / (per[dom]["ms"] * 1e-3) / 1e9 if algo else None
    # DRAM bytes per algorithmic byte from the ncu capture of a smaller case of the same kernel (profiles/), scaled to
    # this step's launches by the bytes they process
    ratio = {"sg_r2_decode": 0.742}.get(dom)
    traffic = ratio * algo / per[dom]["calls"] if ratio and algo else None
    return {"bound": "hbm", "kernel": f"{dom} ({per[dom]['calls']} calls per step)", "achieved": ach, "peak": peak, "peak_kind": peak_kind,
            "unit": "GB/s", "frac": ach / peak if ach else None, "traffic": traffic,
            "traffic_from": "profiles/r2_decode_ncu_full.md: 123.5 MB of DRAM traffic for 166.6 MB of algorithmic bytes on one 4096 x 12288 "
                            "tensor, scaled by the bytes of a launch here" if traffic else None,
            "share_of_device_time": round(per[dom]["ms"] / max(sum(v["ms"] for v in per.values()), 1e-9), 3),
            "note": "the step is bound by the host pipeline (device time is a small part of the wall clock); the kernel-level "
                    "rooflines are under `kernels`"}


def pack_cpu_baseline(args, tmp, quantize, cli):
    """the reference's --cpu path on the bounded sample, in a child process (its kernels and this process's cannot share
    one interpreter); and this library on the same sample, for a like-for-like ratio and an archive comparison"""
    from seedpack_b200 import synthrepo
    try:
        repo = os.path.join(tmp, "sample")
        made = synthrepo.make_repo(repo, SAMPLE, quantize, seed=1, keep_weights=True)
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "1", "--warmup", "0", "--repo-dir", repo],
                           capture_output=True, text=True, timeout=1200, env={k: v for k, v in os.environ.items() if k != "SEEDPACK_CPU"})
        ref_line = json.loads(r.stdout.strip().splitlines()[-1])
        if "unavailable" in ref_line:
            return {"value": None, "unit": "GB/s", "cores": 0, "kind": "reference", "sample": ref_line["unavailable"]}
        arc = os.path.join(tmp, "sample.seedpack")
        _quiet(cli.main, ["pack", "-q", "-f", "-o", arc, repo])
        t0 = time.perf_counter()
        _quiet(cli.main, ["pack", "-q", "-f", "-o", arc, repo])
        _quiet(cli.main, ["test", arc])
        ours = 2 * made["bytes"] / (time.perf_counter() - t0) / 1e9
        out = dict(ref_line["cpu_baseline"])
        out.update(pack_gbs=ref_line["pack_gbs"], unpack_gbs=ref_line["unpack_gbs"], this_library_on_the_sample_gbs=ours,
                   sample_archive_identical=_file_digest(arc) == ref_line["archive_sha256"])
        return out
    except Exception as e:                                   # the baseline is reported, never required
        return {"value": None, "unit": "GB/s", "cores": 0, "kind": "reference", "sample": f"failed: {e}"}



# ------------------------------------------------------------------------------------------------------
# `shard`: one window of a 27B-shaped repository (rows of 5120 and 17408 weights) cut over the ranks by rANS segment:
# every rank regrows the rows behind its segments, compares them with the stored blocks, models and counts its segments;
# counts are added through the host, tables normalised on every rank alike, segments coded and gathered on rank 0.
SHARD_TYPES = [2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 16, 17, 18, 19, 20, 21, 22, 23, 29, 42]


def run_shard(args):
    import hashlib
    import torch
    import torch.distributed as dist
    from seedpack_b200 import shardcode
    from seedpack_b200.qr import BS, QK
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.new_group(backend="gloo")           # the path's own exchange goes through the host
    types = [int(t) for t in args.shard_types.split(",")] if args.shard_types else SHARD_TYPES
    shapes = [(args.shard_rows, 5120), (args.shard_rows // 4, 17408)]
    case = shardcode.make_case(types[0], shapes, seed=11)
    batches = {}
    for T in types:
        b = shardcode.ShardedBatch(dict(case, T=T), rank, world, local, group=group)
        if batches:                                      # the base window and importance vectors are on the device once
            first = next(iter(batches.values()))
            b.seed, b.imx = first.seed, first.imx
        batches[T] = b.prepare()
    nweights = sum(nr * nc for nr, nc in shapes)
    file_bytes = sum(nweights // QK[T] * BS[T] for T in types)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(2)

    def step():
        """every batch of the window; batch k is framed by rank k mod N, in a thread beside the next batch's GPU work.
        -> (SHA-256 over the batches' SHA-256 digests in batch order: the same at every N, bytes that differ)"""
        mine, nd = {}, 0
        for k, T in enumerate(types):
            fut, d = batches[T].run(root=k % world, pool=pool)
            nd += d
            if fut is not None:
                mine[k] = fut
        mine = {k: hashlib.sha256(f.result()).digest() for k, f in mine.items()}
        if world > 1:
            parts = [None] * world if rank == 0 else None
            dist.gather_object(mine, parts, dst=0, group=group)
            if rank != 0:
                return None, nd
            mine = {k: v for p in parts for k, v in p.items()}
        return hashlib.sha256(b"".join(mine[k] for k in range(len(types)))).hexdigest(), nd

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        digest, ndiff = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.summary()
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    if rank == 0:
        peak, peak_kind = peaks()
        ms_step = ms / args.steps
        val = file_bytes / (ms_step * 1e-3) / 1e9
        line = {"metric": "sharded regrow + compare + code, GB/s of GGUF bytes", "value": val, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"one window of a 27B-shaped repository: BF16 tensors {shapes[0][0]}x5120 and {shapes[1][0]}x17408 "
                                       f"({nweights} weights), stored as {len(types)} quant types with another importance vector and ~0.5% "
                                       "of blocks disturbed; per type: regrow, compare, QR-code; cut over the ranks by rANS segment, counts "
                                       "and coded segments exchanged through the host (gloo)",
                           "l2": "inputs larger than L2", "types": types},
                "clocks": clocks, "batches_sha256": digest, "gpu_launches": int(len(types) * 7 * args.steps),
                "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                        "note": "the window and the stored blocks are resident; the host exchange is inside the timed region"},
                "roofline": None, "cpu_baseline": None}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------
# Coder workloads: the rANS symbol coder on a stream of 2^30 residual symbols, the QR residual coder and the
# R2 BF16 base codec on the config-2 tensor.  Kernel times are CUDA-event times of the library calls
# (seedpack_b200._lib.timed); `e2e` is wall time through the Python classes with host buffers on both sides.
def _codec_line(args, metric, workload, unit_bytes, kern_ms, e2e_s, h2d, d2h, table, roof, cpu, launches, clocks):
    peak, peak_kind = peaks()
    roof = dict(roof, peak=peak, peak_kind=peak_kind, unit="GB/s", frac=roof["achieved"] / peak, bound="hbm", traffic=None)
    return {"metric": metric, "value": unit_bytes / (kern_ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": kern_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic", "config": {"workload": workload, "l2": "inputs larger than L2", "kernels": table},
            "clocks": clocks, "e2e": {"value": unit_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "roofline": roof, "cpu_baseline": cpu}


def _timed_steps(args, fn):
    """fn() once per step after the warm-up steps -> ({kernel: ms per step}, wall seconds per step, clocks)"""
    import torch
    from seedpack_b200 import _lib
    for _ in range(max(args.warmup, 1)):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    fn()
    torch.cuda.synchronize()
    one = max(time.perf_counter() - t0, 1e-4)
    steps = max(args.steps, int(1.0 / one) + 1)       # at least a second under load: the clock sampler must see it
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    _lib.timing_start()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / steps
    ms = {k: v / steps for k, v in _lib.timing_stop().items()}
    return ms, wall, sampler.summary()


def synth_symbols(nsym, seed, device):
    """the residual-codec microbenchmark's stream: blocks of 32 symbols, each block with an alphabet of 4 / 5 / 6 / 8 bits and one of
    292 context tables; 97 % zeros, the rest discrete Laplace(b = 2) folded into the alphabet"""
    import torch
    g = torch.Generator(device=device); g.manual_seed(seed)
    nb = nsym // 32
    kind = torch.randint(0, 4, (nb,), generator=g, device=device)
    tab = (kind * 73 + torch.randint(0, 73, (nb,), generator=g, device=device)).to(torch.int16)
    mask = torch.tensor([15, 31, 63, 255], device=device)[kind].to(torch.int32)
    sym = torch.empty(nsym, dtype=torch.uint8, device=device)
    step = 1 << 24
    for a in range(0, nsym, step):
        n = min(step, nsym - a)
        u = torch.rand(n, generator=g, device=device)
        mag = torch.floor(-2.0 * torch.log(torch.rand(n, generator=g, device=device).clamp_min(1e-12))).to(torch.int32)
        sgn = torch.randint(0, 2, (n,), generator=g, device=device, dtype=torch.int32) * 2 - 1
        v = torch.where(u < 0.97, torch.zeros_like(mag), mag * sgn) & mask[a // 32:(a + n) // 32].repeat_interleave(32)
        sym[a:a + n] = v.to(torch.uint8)
    return sym, tab


def run_rans(args):
    import torch
    from seedpack_b200.rans import RansCodec
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    S, NTAB = args.symbols, 294
    sym, tab = synth_symbols(S, 1, dev)
    c = RansCodec(0)
    state = {}

    def step():
        r = c.encode(sym, tab, 32, NTAB)
        out = c.decode(r["stream"], r["off"], tab, 32, S, r["freq"], r["used"], NTAB)
        state.update(r=r, out=out)

    ms, _, clocks = _timed_steps(args, step)
    assert torch.equal(state["out"], sym), "round trip failed"
    coded = state["r"]["total"]
    kern = sum(ms.values())
    algo = {"rans_hist": S + S // 16, "rans_encode": S + S // 16 + coded, "scan_gather": 2 * coded, "rans_decode": coded + S // 16 + S}
    table = {k: {"ms": round(v, 3), "algo_gbs": round(algo[k] / (v * 1e-3) / 1e9, 1)} for k, v in ms.items()}
    dom = max(ms, key=ms.get)
    # end to end: symbols and table ids from pinned host memory, coded stream back; then the stream in, symbols back
    hs, ht = sym.cpu().pin_memory(), tab.cpu().pin_memory()
    hback = torch.empty(S, dtype=torch.uint8).pin_memory()

    def e2e():
        ds, dt_ = hs.to(dev, non_blocking=True), ht.to(dev, non_blocking=True)
        r = c.encode(ds, dt_, 32, NTAB)
        hstream = r["stream"].cpu()                       # padded to the 16-byte windows the decoder reads
        hoff = r["off"].cpu()
        out = c.decode(hstream.to(dev), hoff.to(dev), dt_, 32, S, r["freq"], r["used"], NTAB)
        hback.copy_(out, non_blocking=True)
        torch.cuda.synchronize()

    e2e()
    t0 = time.perf_counter(); e2e(); e2e_s = time.perf_counter() - t0
    # CPU baseline: the plain-C restatement of the same coder, one thread, on the first 4 Mi symbols
    cpu = None
    try:
        from oracle import rans as orans
        n = min(S, 1 << 22)
        hsym, htab = sym[:n].cpu().numpy(), tab[:n // 32].cpu().numpy().view(np.uint16)
        from seedpack_b200.rans import normalize
        counts = np.bincount(np.repeat(htab, 32).astype(np.int64) * 256 + hsym, minlength=NTAB * 256).reshape(NTAB, 256)
        freq, used = normalize(counts)
        full = np.zeros((NTAB, 256), np.uint16); full[used] = freq
        t0 = time.perf_counter()
        st, off = orans.encode(hsym, htab, 32, 16384, full)
        back, _ = orans.decode(st, off, htab, 32, n, 16384, full)
        dtc = time.perf_counter() - t0
        assert np.array_equal(back, hsym)
        cpu = {"value": n / dtc / 1e9, "unit": "GB/s", "cores": 1, "kind": "port", "sample": f"first {n} symbols, encode + decode"}
    except Exception as e:
        cpu = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    line = _codec_line(args, "rANS symbol coder GB/s of symbols, histogram + encode + gather + decode",
                       f"{S} symbols in blocks of 32 with one of {NTAB} tables per block, 97% zeros + Laplace(b=2) on 4/5/6/8-bit alphabets, "
                       f"segments of 16384, 12 probability bits; coded to {coded} bytes",
                       S, kern, e2e_s, S + S // 16 + coded, coded + S, table,
                       {"kernel": dom, "achieved": algo[dom] / (ms[dom] * 1e-3) / 1e9}, cpu, 6, clocks)
    return line


def _flip_bytes(a, bs, frac, seed):
    """one random byte XOR-flipped in `frac` of the blocks of a (residuals that no prediction explains)"""
    rng = np.random.default_rng(seed)
    nb = len(a) // bs
    pick = rng.choice(nb, max(1, int(nb * frac)), replace=False)
    a = a.copy()
    a[pick * bs + rng.integers(0, bs, len(pick))] ^= rng.integers(1, 256, len(pick)).astype(np.uint8)
    return a


def run_qr(args):
    import torch
    from seedpack_b200.gpuquant import GPUQuant
    from seedpack_b200.qr import QRCodec, GRID_TYPES
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    gq, qc = GPUQuant(0), QRCodec(0)
    K = args.tensors
    tens = [synth_tensor(1 + k) for k in range(K)]
    imx = tens[0][1]
    seed_bytes = np.concatenate([b.view(np.uint8).reshape(-1) for b, _ in tens])
    xs = [torch.from_numpy(b.view(np.int16)).to(dev).view(torch.bfloat16).reshape(-1) for b, _ in tens]
    rng = np.random.default_rng(7)
    imx2 = (imx * np.exp(rng.normal(0, 0.3, imx.shape))).astype(np.float32)      # the file was made with another matrix
    types = [int(t) for t in args.qr_types.split(",")]
    table, tot_bytes, tot_ms, tot_wall, launches, dom, clocks = {}, 0, 0.0, 0.0, 0, None, None
    for T in types:
        name, qk, bs = QFUN[T]
        Ps = gq.quantize_tensors(T, [(x, NPR) for x in xs], [imx] * K)
        Fs = [_flip_bytes(f, bs, 0.005, T + 100 * k) for k, f in enumerate(gq.quantize_tensors(T, [(x, NPR) for x in xs], [imx2] * K))]
        ioff = 0 if T in GRID_TYPES else -1
        enc_items = [(Fs[k], Ps[k], k * 2 * NROWS * NPR, 30, NPR, ioff) for k in range(K)]
        dec_items = [(Ps[k], k * 2 * NROWS * NPR, 30, NPR, ioff) for k in range(K)]
        F, P = np.concatenate(Fs), np.concatenate(Ps)
        st = {}

        def step():
            buf = qc.encode(T, enc_items, seed_bytes, imx if T in GRID_TYPES else None)
            out = qc.decode(T, buf, dec_items, seed_bytes, imx if T in GRID_TYPES else None)
            st.update(buf=buf, out=out)

        ms, wall, clocks = _timed_steps(args, step)
        assert np.array_equal(st["out"].cpu().numpy(), F), f"type {T}: round trip failed"
        nfile, coded = len(F), len(st["buf"])
        nw = NROWS * NPR * K
        algo = {"residual_blocks": 2 * nfile, "qr_hist": 2 * nfile + 2 * nw, "qr_encode": 2 * nfile + 2 * nw + coded,
                "qr_stage": 2 * nfile + 2 * nw, "qr_stage_hist": 2 * nfile + 2 * nw, "qr_stage_encode": 2 * nfile + 2 * nw + coded,
                "scan_gather": 2 * coded, "qr_decode": 2 * nfile + 2 * nw + coded}
        kern = sum(ms.values())
        table[name] = {"file_bytes": nfile, "coded_bytes": coded, "differing_blocks": float(np.mean(np.any((F != P).reshape(-1, bs), axis=1))),
                       "ms": {k: round(v, 3) for k, v in ms.items()},
                       "algo_gbs": {k: round(algo[k] / (v * 1e-3) / 1e9, 1) for k, v in ms.items()}, "e2e_s": round(wall, 4)}
        k = max(ms, key=ms.get)
        if dom is None or ms[k] > dom[1]:
            dom = (f"{k} {name}", ms[k], algo[k])
        tot_bytes += nfile; tot_ms += kern; tot_wall += wall; launches += 6
    line = _codec_line(args, "QR residual coder GB/s of tensor bytes, block compare + histogram + encode + gather + decode",
                       f"one coding batch per type ({', '.join(QFUN[t][0] for t in types)}) of {K} tensors of {NROWS}x{NPR}: file quantised with a "
                       "perturbed importance matrix and 0.5% of blocks with a flipped byte, prediction with the plain matrix, BF16 seed",
                       tot_bytes, tot_ms, tot_wall, 2 * tot_bytes + 2 * NROWS * NPR * K * len(types), tot_bytes, table,
                       {"kernel": dom[0], "achieved": dom[2] / (dom[1] * 1e-3) / 1e9},
                       {"value": None, "unit": "GB/s", "cores": 0, "kind": "port",
                        "sample": "no CPU restatement of the QR model is kept; parity is pinned on the reference's own coded batches"},
                       launches, clocks)
    return line


def run_r2(args):
    """the R2 base codec on a file of K tensors of the benchmark shape: the reference's BF16v2 / R2Tensors classes over the
    bound kernels (seedpack_b200.refbind); kernel times are CUDA-event times of the library calls"""
    import torch
    from seedpack_b200 import _lib, refbind, synthrepo
    torch.cuda.set_device(0)
    refbind.install()
    from seedpack import bf16v2, codecs_gguf
    K = args.tensors
    tens = [synth_tensor(1 + k)[0] for k in range(K)]
    data = synthrepo.gguf_bytes([("general.alignment", 4, 32)],
                                [(f"blk.{k}.ffn_up.weight", (NPR, NROWS), 30, NROWS * NPR * 2, (lambda k=k: tens[k])) for k in range(K)])
    n = K * NROWS * NPR * 2
    st = {}

    def step():
        chunk = b"".join(bytes(p) for p in bf16v2.BF16v2().compress_parts(data))
        st.update(chunk=chunk, back=bf16v2.BF16v2().decompress(chunk))

    for _ in range(max(args.warmup, 1)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    _lib.timing_start(calls=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / args.steps
    ms = {k[3:]: v / args.steps for k, v in _lib.timing_stop().items()}
    clocks = sampler.summary()
    assert np.array_equal(np.asarray(st["back"]), np.frombuffer(data, np.uint8)), "round trip failed"
    coded = len(codecs_gguf.unpack(st["chunk"])["stream"])
    algo = {"r2_stats": 3 * n, "row_hash": n, "r2_hist": n, "r2_encode": n + coded, "scan_gather": 2 * coded, "r2_decode": coded + n}
    table = {k: {"ms": round(v, 3), "algo_gbs": round(algo[k] / (v * 1e-3) / 1e9, 1) if k in algo else None} for k, v in ms.items()}
    dom = max((k for k in ms if k in algo), key=ms.get)
    line = _codec_line(args, "R2 BF16 base codec GB/s of BF16 bytes, statistics + row hashes + histogram + encode + gather + decode",
                       f"a GGUF file of {K} BF16 tensors of {NROWS}x{NPR} of one role ({n} bytes), coded to {coded} stream bytes",
                       n, sum(ms.values()), wall, n + coded, coded + n, table, {"kernel": dom, "achieved": algo[dom] / (ms[dom] * 1e-3) / 1e9},
                       {"value": None, "unit": "GB/s", "cores": 0, "kind": "port",
                        "sample": "no CPU restatement of the R2 codec is kept; parity is pinned on the reference's own coded parts"},
                       8, clocks)
    return line


def quant_roofline(name, row, ach_gbs, hbm_peak, peak_kind, fp32_peak):
    """the launch with the largest share of the step, against the roofline that bounds it"""
    traffic = NCU_TRAFFIC.get(name) if NROWS == 4096 else None
    if row["bound"] == "hbm":
        return {"bound": "hbm", "kernel": f"k_quant {name} (largest share of the step)", "achieved": ach_gbs, "peak": hbm_peak,
                "peak_kind": peak_kind, "unit": "GB/s", "frac": ach_gbs / hbm_peak, "traffic": traffic}
    return {"bound": "fp32_issue", "kernel": f"k_quant {name} (largest share of the step)", "achieved": row["fp32_tops"], "peak": round(fp32_peak, 2),
            "peak_kind": "148 SMs x 128 fp32 lanes x sampled SM clock (no FMA: one add or mul per lane and cycle)", "unit": "Tops/s",
            "frac": row["fp32_frac"], "traffic": traffic, "hbm_gbs": round(ach_gbs, 1), "issue_slots_busy": row["issue_slots_busy"],
            "ops_per_weight": OPS[name][0], "instructions_per_weight": OPS[name][1],
            "counted": "fp32 add / mul thread instructions per weight from ncu (profiles/quant_fp32_ops_ncu.md)"}


def case_name(t, use):
    return f"{QFUN[t][0]}{'+imx' if use else ''}"


def main():
    global NROWS, CASES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-rows", type=int, default=0, help="rows of the tensor the CPU baseline quantises per step")
    ap.add_argument("--rows", type=int, default=NROWS, help="rows of the tensor (profiling captures use fewer)")
    ap.add_argument("--only", default="", help="comma-separated launch names to keep, e.g. q4_K+imx,iq2_xs+imx")
    ap.add_argument("--workload", default="pack", choices=["pack", "quant", "shard", "rans", "qr", "r2"],
                    help="pack: pack + test of a synthetic repository (the headline); quant: the quantiser sweep; rans / qr / r2: the coders, one GPU")
    ap.add_argument("--shard-rows", type=int, default=8192, help="shard: rows of the 5120-column tensor (the 17408-column one has a quarter)")
    ap.add_argument("--shard-types", default="", help="shard: comma-separated ggml type ids (default: the 20 types of the reference's table)")
    ap.add_argument("--no-kernels", action="store_true", help="pack: leave the kernel-level workloads out of the line")
    ap.add_argument("--repo", default="c1", help="pack: synthetic repository (a key of seedpack_b200.synthrepo.CONFIGS)")
    ap.add_argument("--without-base", default="no", choices=["no", "all", "q8"],
                    help="pack: remove the BF16 file before packing (all: every quant file stays; q8: the Q8_0 file alone) - a side line, "
                         "not the benchmark's workload")
    ap.add_argument("--repo-dir", default="", help="--impl reference: an existing repository directory to pack instead of making the sample")
    ap.add_argument("--symbols", type=int, default=1 << 30, help="rans: symbols in the stream")
    ap.add_argument("--tensors", type=int, default=4, help="qr / r2: tensors of the benchmark shape in the batch / file")
    ap.add_argument("--qr-types", default="8,12,14,17,18", help="qr: ggml type ids, one coding batch each")
    args = ap.parse_args()
    NROWS = args.rows
    if args.only:
        keep = set(args.only.split(","))
        CASES = [c for c in CASES if case_name(*c) in keep]
        assert CASES, "no such launch"
    if args.workload == "pack":
        (run_reference_pack if args.impl == "reference" else run_pack)(args)
    elif args.workload == "shard":
        run_shard(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload != "quant":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"rans": run_rans, "qr": run_qr, "r2": run_r2}[args.workload](args)))
    else:
        line = run_ours(args)
        if line is not None:
            print(json.dumps(line))


if __name__ == "__main__":
    main()
