"""The reference arm of bench.py runs on host cores only (the oracle port of the reference's CPU
path): it must work without a GPU and print the agreed JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "1", "--cpu-protocol", "quick"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "nvfp4_gemv_hbm_gbps"
    assert line["unit"] == "GB/s" and line["higher_is_better"] is True and line["value"] > 0
    assert line["config"]["workload"] == "gemv_497_mix_27b"
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["sample"]
    assert cb["value"] == line["value"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["h2d_bytes_per_step"] == 0 == e2e["d2h_bytes_per_step"]
    # both arms describe the workload with the same dictionary
    sys.path.insert(0, ROOT)
    import bench

    assert line["config"] == bench.common_config(1)
    proto = line["cpu_protocol"]
    assert len(proto["rows"]) == len(bench.CPU_SHAPES) and proto["mix_497_lower_bound_s"] > 0
