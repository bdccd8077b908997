"""The measurement harness's output contract: one JSON line with the agreed keys, for both arms."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config"}


def _run(*args, timeout=900):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=timeout,
                       cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line(pkg, oracle_mod):
    """`--impl reference`: the reference's CPU SGEMM on a bounded row sample; no GPU needed."""
    d = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert BASE_KEYS <= set(d) and d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["value"] > 0 and d["vs_baseline"] is None and d["dtype"] == "f32"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == pytest.approx(d["value"])
    assert "rows" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]
    # the formula: flops of the step's row sample over its time (a dense CPU SGEMM takes the same time at every
    # density, so its dense-equivalent rate is the same for one density or for the sweep of four)
    rows = int(d["config"]["sample"].split()[0])
    assert d["value"] == pytest.approx(2.0 * rows * 4096 * 4096 / (d["ms_per_step"] * 1e-3) / 1e12, rel=1e-6)
    assert d["metric"].startswith("dense-equivalent TFLOP/s at 4096^3 FP32")


@pytest.mark.gpu
def test_product_arm_line(pkg, cuda):
    d = _run("--steps", "3", "--warmup", "3", "--no-cpu", "--no-scaling-base")
    assert BASE_KEYS <= set(d) and "impl" not in d and d["n_gpus"] == 1 and d["steps"] == 3 and d["dtype"] == "f32"
    assert d["value"] == pytest.approx(4 * 2.0 * 4096 ** 3 / (d["ms_per_step"] * 1e-3) / 1e12, rel=1e-6)
    rf = d["roofline"]
    assert rf["unit"] == "TFLOP/s" and 0.3 < rf["frac"] < 1.1 and rf["frac"] == pytest.approx(rf["achieved"] / rf["peak"])
    assert rf["traffic"] > 201e6                     # at least the compulsory bytes
    assert d["gpu_launches"] == 3 * 4 * 2
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] == 4 * 4 * 4096 * 4096 and e["d2h_bytes_per_step"] == 4 * 4 * 4096 * 4096
    assert 0 < e["value"] < d["value"]               # copies inside: slower than the device-resident number
    assert set(d["sweep"]) == {"11111111", "11110000", "11000000", "10000000"}
    for row in d["sweep"].values():
        assert row["ms_cublas"] > 0 and row["ms_total"] >= row["ms_gemm"] * 0.98
    assert d["clocks"]["sm_max_mhz"] >= d["clocks"]["sm_mhz"] > 0 and isinstance(d["clocks"]["reasons"], list)
    assert d["cpu_baseline"] is None and d["scaling_base"] is None      # both skipped by the flags above
    # comparison columns kept inside `config`: [ours, cuBLAS, reference kernel id 29] in ms per density
    import oracle
    for pat, (ours, cublas, ref29) in d["config"]["ms_ours_cublas_ref29"].items():
        assert ours > 0 and cublas > 0
        if oracle.have_ref():
            assert ref29 > ours, pat                  # the recompiled reference kernel is the bar to beat
    assert len(d["other_configs"]) == 8 and any(k.startswith("c4 M=16") for k in d["other_configs"])
    for row in d["other_configs"].values():
        assert row["ms_total"] > 0 and 0 < row["joint_density"] < 1
