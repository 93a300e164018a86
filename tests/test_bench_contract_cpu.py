"""The benchmark's command-line contract that can be checked without a GPU: the reference arm
answers with one JSON line and exit code 0 when the reference cannot be installed."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec.get("unavailable"), str) and rec["unavailable"]


def test_build_entry_point_compiles_and_imports():
    import importlib.util
    spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(ROOT, "__graft_entry__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()                                   # nvcc cross-compiles for sm_100a without a GPU
    assert os.path.exists(os.path.join(ROOT, "dizo_b200", "ops", "libdizo_b200.so"))
