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
