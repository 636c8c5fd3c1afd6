"""The benchmark's command-line contract, as far as it can be checked without a GPU: the reference arm (the CPU restatement of
the reference's float32 path, bounded sample) prints one JSON line with the agreed keys; the product arm either runs on a GPU
and says how many of the library's kernels it launched, or fails loudly -- it never prints a number computed on the CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_the_agreed_line():
    res = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype", "data",
                "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "int8_quantized_matmul_tops" and line["unit"] == "TOPS" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["warmup"] >= 3
    assert "workload" in line["config"] and "model" not in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1 and base["sample"] and base["value"] == line["value"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_product_arm_never_falls_back_to_the_cpu():
    res = _run("--steps", "3", "--warmup", "3", "--no-gpt", "--short")
    if res.returncode == 0:        # a GPU is present: the line must come from the library's kernels
        line = json.loads(res.stdout.strip().splitlines()[-1])
        assert line.get("impl", "ns_b200") != "reference" and line["gpu_launches"] > 0 and line["roofline"]["achieved"] > 0
    else:
        assert "ns_device_open failed" in res.stderr or "libns_b200.so is missing" in res.stderr, res.stderr[-2000:]
        assert not res.stdout.strip().startswith("{"), "no result line may be printed without a GPU"
