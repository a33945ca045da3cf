"""bench.py's reference arm runs without a GPU: its JSON line must carry the keys the benchmark contract names."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    from oracle import ref
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0", "--ref-rows", "8"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
              "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert k in line, k
    assert line["impl"] == "reference" and line["value"] > 0 and "workload" in line["config"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "reference"


def test_extra_golden_equals_reference_c_code():
    """the committed vectors of the five further types are what oracle/_ref produces"""
    from oracle import ref
    from tests import synth
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    g = np.load(os.path.join(ROOT, "tests", "golden", "quant_extra_golden.npz"))
    x = synth.bf16_bits_to_f32(g["bits"]).reshape(int(g["nrows"]), int(g["npr"]))
    for t in sorted(ref.EXTRA):
        y = ref.quantize(t, x, None, threads=1)
        assert np.array_equal(y, g[f"q_{t}"]), t
        assert np.array_equal(ref.dequantize(t, y, x.size).view(np.uint32), g[f"d_{t}"].view(np.uint32)), t


def test_pack_config_names_the_workload():
    """both arms print the same `config`; the side lines without the BF16 file say so in it"""
    sys.path.insert(0, ROOT)
    import bench
    base = bench.pack_config("c1", 1)
    assert "0.5% of blocks disturbed" in base["workload"] and "one repository per GPU" not in base["workload"]
    assert bench.pack_config("c1", 8)["workload"].endswith("one repository per GPU")
    assert "Q8_0 file alone" in bench.pack_config("c1", 1, "q8")["workload"] and "BF16 file removed" in bench.pack_config("c1", 1, "all")["workload"]
    assert bench.pack_config("c1", 1, "no") == base
