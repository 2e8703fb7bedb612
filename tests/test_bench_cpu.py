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


def test_numa_binding_reads_a_fake_sysfs(tmp_path):
    """bench.bind_to_gpu_numa_node against a made-up /sys: two nodes, the GPU on node 1 whose CPUs include the
    ones this process may use; with one node, an unknown node or foreign CPUs it leaves the affinity alone."""
    sys.path.insert(0, ROOT)
    import bench

    class Props:
        pci_domain_id, pci_bus_id, pci_device_id = 0, 0x1b, 0

    class FakeTorch:
        class cuda:
            @staticmethod
            def get_device_properties(i):
                return Props()

    mine = sorted(os.sched_getaffinity(0))
    before = os.sched_getaffinity(0)

    def make(root, node_of_gpu, node1_cpus, n_nodes=2):
        for n in range(n_nodes):
            d = root / "devices/system/node" / f"node{n}"
            d.mkdir(parents=True)
            (d / "cpulist").write_text(node1_cpus if n == 1 else "4000-4003")
        dev = root / "bus/pci/devices/0000:1b:00.0"
        dev.mkdir(parents=True)
        (dev / "numa_node").write_text(f"{node_of_gpu}\n")

    try:
        a = tmp_path / "a"; make(a, 1, f"{mine[0]}-{mine[0]},5000-5003")
        note = bench.bind_to_gpu_numa_node(FakeTorch, 0, sysfs=str(a))
        assert note and "NUMA node 1" in note and os.sched_getaffinity(0) == {mine[0]}
        os.sched_setaffinity(0, before)
        b = tmp_path / "b"; make(b, -1, "0-3")
        assert bench.bind_to_gpu_numa_node(FakeTorch, 0, sysfs=str(b)) is None
        c = tmp_path / "c"; make(c, 1, "5000-5003")
        assert bench.bind_to_gpu_numa_node(FakeTorch, 0, sysfs=str(c)) is None
        d = tmp_path / "d"; make(d, 0, "0-3", n_nodes=1)
        assert bench.bind_to_gpu_numa_node(FakeTorch, 0, sysfs=str(d)) is None
        assert bench.bind_to_gpu_numa_node(FakeTorch, 0, sysfs=str(tmp_path / "missing")) is None
        assert os.sched_getaffinity(0) == before
        assert bench._parse_cpulist("0-2,8,10-11\n") == {0, 1, 2, 8, 10, 11}
    finally:
        os.sched_setaffinity(0, before)
