"""The benchmark's reference arm (`bench.py --impl reference`) needs no GPU: it times the reference's own CPU expert
kernels on a bounded sample of the default workload.  This checks that the arm runs and that its JSON line carries the
keys the contract names, with the main arm's metric and unit."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libstrata_ref.so")):
        pytest.skip("the compiled reference checker is absent (no reference checkout at build time)")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--cpu-seconds", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert line["metric"] == "MoE layer tokens/s" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["n_gpus"] == 1
    assert line["config"]["workload"].startswith("c3")
    base = line["cpu_baseline"]
    assert base["kind"] == "reference" and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
