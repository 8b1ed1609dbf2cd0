"""bench.py's contract where no GPU is needed: the reference arm (the CPU restatement on host
cores) prints one JSON line with the agreed keys, and the product arm refuses to run without a
CUDA device instead of falling back to anything."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=600, env=env, cwd=ROOT)


def test_reference_arm_prints_the_agreed_line():
    r = run("--impl", "reference", "--steps", "1", "--warmup", "0", "--reference-seconds", "0.5")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "gemm_f16_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["steps"] == 1 and line["warmup"] == 0
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["config"]["workload"] == "gemm_f16_16384x16384x8192"
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and "rows 0.." in cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_product_arm_has_no_cpu_fallback():
    r = run("--steps", "1", "--warmup", "1", "--no-extras", "--no-cpu", "--min-time", "0")
    assert r.returncode != 0
    assert "no CUDA device" in (r.stderr + r.stdout)
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
