"""The reference arm of bench.py runs without a GPU: one JSON line with the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "fused_gemm_tflops" and d["unit"] == "TFLOP/s"
    assert d["steps"] == 1 and d["warmup"] == 1           # the counts it printed are the counts it timed
    assert d["value"] > 0 and d["vs_baseline"] is None and "workload" in d["config"]
    # the product arm prints the same `config` object for this workload and rank count
    sys.path.insert(0, ROOT)
    import bench
    assert d["config"] == bench.config_for("c4", 1)
    assert d["config"]["tokens_per_gpu"] == 8192 and d["config"]["sharding"] == "tokens"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]


def test_reference_arm_covers_every_single_gpu_configuration():
    """The arm asserts by itself that the CUDA library is not mapped into its process."""
    for wl, metric in (("c2", "pointwise_permute_hbm_gbs"), ("c1", "train_steps_per_s")):
        out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", wl, "--steps", "2", "--warmup", "1"],
                             capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert out.returncode == 0, out.stderr[-2000:]
        d = json.loads(out.stdout.strip().splitlines()[-1])
        assert d["metric"] == metric and d["steps"] == 2 and d["value"] > 0


def test_product_arm_refuses_to_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode != 0 and "no CPU path" in (out.stderr + out.stdout)
