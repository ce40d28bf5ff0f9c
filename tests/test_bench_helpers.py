"""Host-side pieces of bench.py that need no GPU: the lookup that ties roofline.traffic to the
ncu capture of the very kernel that ran, the configuration block, and the CPU arms."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def _table():
    return json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())["kernels"]


def test_every_capture_names_the_code_it_was_taken_from():
    for entry in _table():
        assert entry["code"].startswith("#") and len(entry["code"]) == 9, entry
        assert (ROOT / "profiles" / entry["source"]).exists(), entry
        assert entry["code"] in (ROOT / "profiles" / entry["source"]).read_text(), entry


def test_traffic_is_used_only_for_the_kernel_version_that_was_captured():
    entry = next(e for e in _table() if e["match"] == "flat 2d vec2 in4 out2 red1")
    kernel = {"kernel": f"group33[flat 2d vec2 in4 out2 red1] {entry['code']}", "gbs": 6000.0, "ms_per_launch": 0.5}
    traffic, source = bench.dram_traffic(kernel)
    algorithmic = 6000.0e9 * 0.5e-3
    assert traffic == pytest.approx(entry["dram_bytes_per_algorithmic_byte"] * algorithmic)
    assert source == "profiles/" + entry["source"]
    # the same kernel after any change to its source, the device header or its tile configuration
    stale = dict(kernel, kernel="group33[flat 2d vec2 in4 out2 red1] #00000000")
    traffic, why = bench.dram_traffic(stale)
    assert traffic is None and "another version" in why
    traffic, why = bench.dram_traffic({"kernel": "group1[strided 2d vec1 in3 out1 red0] #12345678", "gbs": 1.0,
                                       "ms_per_launch": 1.0})
    assert traffic is None and "no capture" in why


def test_config_block_is_the_same_for_both_arms():
    a = bench.config_for("jacobi2d", 4, 1.0, 64)
    assert a["halo_depth"] == 64 and a["parallelism"] == "slab4" and "8192x2048" in a["workload"]
    b = bench.config_for("cg", 1, 1.0, 1)
    assert b["halo_depth"] == 0 and "8192x8192" in b["workload"]


@pytest.mark.parametrize("workload", ["cg", "jacobi2d"])
def test_reference_arm_prints_one_line_with_both_cpu_layouts(workload):
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", workload,
                          "--scale", "0.03125", "--steps", "4", "--warmup", "3"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["steps"] == 4 and line["warmup"] == 3
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"] and line["gpu_launches"] == 0
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"]
    assert base["tiled"]["value"] > 0 and base["tiled"]["tiles"] >= 1
