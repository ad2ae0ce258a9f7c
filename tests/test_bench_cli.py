"""The benchmark's CPU-only legs, run as the driver runs them (a subprocess, one JSON line on stdout)."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300, env=e)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout.strip().splitlines()


def test_reference_arm_prints_one_line_with_the_contract_keys():
    """`--impl reference` on the smallest configuration: one JSON line, the reference's own function when the
    copy under oracle/_ref is importable (kind "reference"), else the oracle port with the reason."""
    lines = _run("--impl", "reference", "--workload", "fp8_tensor", "--steps", "1", "--warmup", "1")
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0
    base = d["cpu_baseline"]
    assert base["cores"] >= 1 and "4096 of 4096 rows" in base["sample"]
    have_copy = os.path.isfile(os.path.join(ROOT, "oracle", "_ref", "transformer_nuggets", "fp8", "scaled_quant.py"))
    assert base["kind"] == ("reference" if have_copy else "port")
    if not have_copy:
        assert "not importable" in base["sample"]


def test_reference_arm_is_silent_on_other_ranks():
    assert _run("--impl", "reference", "--workload", "fp8_tensor", "--steps", "1", "--warmup", "1", env={"RANK": "1"}) == []


def test_traffic_record_is_read_from_the_profile_data_file():
    sys.path.insert(0, ROOT)
    import bench

    r = bench.measured_traffic("k_cast", 1 << 20)
    with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
        rec = json.load(f)["k_cast"]
    per_elem = (rec["dram_bytes_read"] + rec["dram_bytes_write"]) / rec["elements"]
    assert abs(r["traffic"] - per_elem * (1 << 20)) < 1e-6 and 2.0 < r["traffic_bytes_per_element"] < 3.5
    assert bench.measured_traffic("no_such_kernel", 10)["traffic"] is None
