#!/usr/bin/env python
"""Quantiser sweep benchmark (BASELINE config 2): one BF16 tensor of 4096 x 12288 seeded weights plus a
12288-entry importance matrix, re-quantised into every ggml type the path handles.

A step = one pass over the tensor for every type: the 20 types with the importance matrix, then the 15
types whose matrix-free routine is a different code path.  Metric: GB/s of GGUF (quantised) bytes regrown.

    python bench.py --gpus N --steps K --warmup W          (this repo's CUDA path)
    python bench.py --impl reference ...                   (the reference's own C quantisers on the host cores)

Multi-GPU: the path shards by tensor / row-block with no exchange; every rank quantises its own tensor
of the full size (weak scaling), timed on the device, maximum over ranks.
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
        22: ("iq2_s", 256, 82), 23: ("iq4_xs", 256, 136), 29: ("iq1_m", 256, 56), 42: ("q2_0", 64, 18)}
NO_IMX_TOO = [2, 3, 6, 7, 10, 11, 12, 13, 14, 18, 20, 21, 22, 23, 29]     # types whose matrix-free routine differs
CASES = [(t, True) for t in sorted(QFUN)] + [(t, False) for t in NO_IMX_TOO]


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
    cfg = {"workload": workload_text(), "sample_rows": rows}
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
                             "sample": f"first {rows} of {NROWS} rows of the same tensor, all {len(CASES)} launches per step"},
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
    if world > 1:
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
    hout = torch.empty(max(quant_bytes(t) for t, _ in CASES) + 64, dtype=torch.uint8).pin_memory()

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

    # end to end through the public API: host BF16 + importance matrix in, quantised bytes out to the host
    def e2e_step():
        xd = hx.to(dev, non_blocking=True).view(torch.bfloat16).reshape(-1)
        wd = himx.to(dev, non_blocking=True)
        for t, use in CASES:
            y = gq.quantize_tensors(t, [(xd, NPR)], [wd if use else None], device=True)[0]
            hout[:y.numel()].copy_(y, non_blocking=True)
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
        for k, (t, use) in enumerate(CASES):
            a = algo_bytes(t, use) / (per_ms[k] * 1e-3) / 1e9
            table[f"{QFUN[t][0]}{'+imx' if use else ''}"] = {"ms": round(float(per_ms[k]), 4), "algo_gbs": round(a, 1),
                                                              "gguf_gbs": round(quant_bytes(t) / (per_ms[k] * 1e-3) / 1e9, 2),
                                                              "hbm_frac": round(a / peak, 4)}
        dom = int(np.argmax(per_ms))
        dt, duse = CASES[dom]
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
                           "l2": "flushed between launches (256 MiB memset inside the timed region)",
                           "per_type": table},
                "clocks": clocks,
                "e2e": {"value": world * out_bytes / e2e_s / 1e9, "unit": "GB/s",
                        "h2d_bytes_per_step": int(hx.numel() * 2 + himx.numel() * 4), "d2h_bytes_per_step": int(out_bytes)},
                "gpu_launches": int(launches),
                "roofline": {"bound": "hbm", "kernel": f"k_quant {QFUN[dt][0]}{'+imx' if duse else ''} (largest share of the step)",
                             "achieved": ach, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": ach / peak, "traffic": None},
                "cpu_baseline": cpu}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


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
    args = ap.parse_args()
    NROWS = args.rows
    if args.only:
        keep = set(args.only.split(","))
        CASES = [c for c in CASES if case_name(*c) in keep]
        assert CASES, "no such launch"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
