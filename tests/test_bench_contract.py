"""The benchmark's reference arm runs on the host cores (no GPU): its one JSON line must carry the keys the contract
names, and the workload table must be self-consistent."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["value"] > 0 and d["steps"] == 1
    assert d["vs_baseline"] is None and d["data"] == "synthetic" and "workload" in d["config"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
    # the other configurations ride along, each with its own CPU value
    assert set(d["workloads"]) == {"c1", "c3", "c4", "c5", "meta", "fused", "next"}
    for rec in d["workloads"].values():
        assert rec["value"] > 0 and rec["unit"] in ("GB/s", "TFLOP/s") and rec["kind"] == "port" and rec["sample"]


def test_workload_tables_are_consistent():
    sys.path.insert(0, ROOT)
    import bench
    assert set(bench.WORKLOADS) == {"c1", "c2", "c3", "c4", "c5", "meta", "fused", "next"}
    assert bench.HEADLINE == "c2" and set(bench.CONFIGS) == {"c1", "c3", "c4", "c5", "meta", "fused", "next"}
    for key, cls in bench.WORKLOADS.items():
        wl = cls()
        parts = set(wl.work())
        assert parts == set(wl.launches) == set(wl.kernel_of), key
        assert set(getattr(wl, "traffic", {})) <= parts
        assert set(getattr(wl, "all_reduced", ())) <= parts
        assert wl.unit in ("GB/s", "TFLOP/s") and wl.bound in ("hbm", "tensor") and wl.scaling in ("weak", "strong")
