"""The benchmark entry points that must work without a GPU: the reference arm's one-line answer and the
build / smoke module's surface."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-1000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    row = json.loads(lines[0])
    assert row["impl"] == "reference" and isinstance(row.get("unavailable"), str) and row["unavailable"]


def test_entry_module_exposes_build_and_smoke():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    assert callable(g.build) and callable(g.smoke)
    g.build()                                     # a no-op when the content hashes match
    from flexkv_b200 import _native
    assert os.path.dirname(_native.C.__file__) == os.path.join(ROOT, "flexkv_b200")     # in-tree, not site-packages


def test_worker_benchmark_runs_on_the_cpu_data_plane(tmp_path):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "benchmark_workers.py"), "--device", "cpu",
                          "--blocks", "8", "--iters", "1", "--warmup", "1", "--ssd-dir", str(tmp_path / "ssd"),
                          "--out", str(tmp_path / "rows.json")], capture_output=True, text=True, timeout=200)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-1500:]
    rows = json.loads((tmp_path / "rows.json").read_text())
    assert [r["type"] for r in rows] == ["D2H", "H2D", "H2DISK", "DISK2H"]
    assert all(r["bytes"] == 8 * 2097152 and r["gbs"] > 0 for r in rows)


def test_standalone_example_runs_on_the_cpu_data_plane():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "standalone_roundtrip.py"), "--device", "cpu",
                          "--tokens", "128"], capture_output=True, text=True, timeout=200)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-1500:]
    assert "bytes identical=True" in out.stdout
