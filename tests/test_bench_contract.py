"""The benchmark's reference arm on CPU (no GPU needed): it runs the oracle over a whole token step and prints one JSON
line with the contract's keys, the same `config` the product arm prints for the same command line, and the marks of a
CPU arm (impl, cpu_baseline, an e2e block without copies)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--layers", "1", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["higher_is_better"] is True
    assert line["steps"] == 1 and line["n_gpus"] == 1 and line["vs_baseline"] is None
    assert line["value"] > 0 and abs(line["ms_per_step"] * line["value"] - 1000.0) < 1e-6 * 1000.0
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and "measured" in cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the workload description is the product arm's for the same command line
    sys.path.insert(0, ROOT)
    import bench
    from ingot_b200.chain import QWEN3_8B
    want = bench.workload_config(QWEN3_8B, 1, 1, 1, line["config"].get("bytes", 0) or 0)
    assert line["config"]["workload"] == want["workload"] and line["config"]["layers"] == 1
    assert set(line["config"]) == set(want)
