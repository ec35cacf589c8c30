"""The reference arm of bench.py runs on CPU and prints one JSON line with the
keys the benchmark contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload",
                          "tf32_4096", "--steps", "1", "--warmup", "0"], capture_output=True, text=True,
                         timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["metric"] == "TF32 GEMM TFLOPS @4096^3" and d["dtype"] == "tf32" and d["data"] == "synthetic"
    assert d["config"]["workload"] == "tf32_4096" and "model" not in d["config"]
    assert d["vs_baseline"] is None and d["steps"] == 1 and d["n_gpus"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "rows of A" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_reference_arm_uses_the_affinity_mask_not_omp_num_threads():
    """torchrun sets OMP_NUM_THREADS=1 for every rank; the reference arm must
    still use every host thread the process may run on, or its number (and any
    ratio against it) is off by the core count."""
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--workload", "tf32_4096", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    d = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][0])
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert d["n_gpus"] == 2 and d["impl"] == "reference"


def test_bench_defaults_and_workloads():
    """The line's extra objects are on by default and every profile case names a
    workload the harness can build (no GPU needed to check the tables)."""
    sys.path.insert(0, ROOT)
    import bench
    assert set(bench.ALSO) <= set(bench.WORKLOADS) and "cfg5" in bench.WORKLOADS
    assert bench.WORKLOADS["cfg5"][1:4] == (32768, 65536, 8192)
    assert bench.tolerance("bf16", 8192, 1.0, 1.0) == 1e-5 * 8192 ** 0.5
    assert bench.tolerance("tf32", 4096, 1.0, 1.0) == 5e-5 * 4096 ** 0.5
    assert bench.tolerance("tf32", 2048, 1.0, 1.0) == 1e-5 * 2048 ** 0.5
    r = bench.roofline_of("bf16", 128, 8192, 8192, 0.045, bench.measured_peaks(), None)
    assert r["bound"] == "hbm" and 0 < r["frac"] < 1
    r = bench.roofline_of("bf16", 8192, 8192, 8192, 0.68, bench.measured_peaks(), 1.0e9)
    assert r["bound"] == "tensor" and r["traffic"] == 1.0e9 and r["algorithmic_bytes"] == 536870912
