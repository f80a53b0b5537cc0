"""bench.py's output contract, as far as it can be checked without a GPU: the reference arm runs on the host cores, so its
JSON line is produced here; the GPU arm's line is checked for its helpers only."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*flags):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines  # standard output carries the JSON line and nothing else
    return json.loads(lines[0])


def test_reference_arm_prints_one_line_with_the_contract_keys():
    r = run_bench("--impl", "reference", "--workload", "c1", "--steps", "1", "--warmup", "0")
    assert r["impl"] == "reference" and r["higher_is_better"] is True and r["vs_baseline"] is None
    assert r["metric"].startswith("train samples/sec") and r["unit"] == "samples/s" and r["value"] > 0
    assert r["n_gpus"] == 1 and r["steps"] == 1 and r["warmup"] == 0 and r["data"] == "synthetic"
    cb = r["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == r["value"] and isinstance(cb["sample"], str) and cb["sample"]
    assert r["e2e"] == {"value": r["value"], "unit": r["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert r["config"]["workload"].startswith("c1: ") and json.loads(r["config"]["workload"][4:])["kind"] == "mlp"


def test_both_arms_name_the_workload_the_same_way():
    sys.path.insert(0, ROOT)
    try:
        import bench
    finally:
        sys.path.remove(ROOT)
    for name, cfg in bench.WORKLOADS.items():
        if cfg.get("kind") == "gemm":
            continue
        s = bench.workload_string(name, cfg)
        assert s.startswith(name + ": ")
    assert bench.workload_string("c4", bench.WORKLOADS["c4"]) == "c4: " + json.dumps(bench.WORKLOADS["c4"])


def test_gemm_traffic_figure_belongs_to_the_committed_gemm_source():
    """roofline.traffic is an ncu measurement stored with the SHA-256 of the GEMM source it was taken with; a changed
    kernel must come with a new capture (the command is in the comment above bench.GEMM_TRAFFIC's definition), or the
    bench line reports null with the reason instead of a stale number."""
    sys.path.insert(0, ROOT)
    try:
        import bench
    finally:
        sys.path.remove(ROOT)
    per_launch, why = bench.gemm_traffic(12)
    assert per_launch is not None, why
    assert 30e6 < per_launch < 100e6
    saved = bench.GEMM_TRAFFIC["kernel_sha256"]
    bench.GEMM_TRAFFIC["kernel_sha256"] = "0" * 64
    try:
        assert bench.gemm_traffic(12)[0] is None
    finally:
        bench.GEMM_TRAFFIC["kernel_sha256"] = saved
