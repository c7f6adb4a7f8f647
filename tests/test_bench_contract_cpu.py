"""The command-line contract of bench.py that does not need a GPU: the reference arm answers with one JSON line
and exit code 0, and the entry module exposes build() and smoke()."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps",
                        "2", "--warmup", "1"], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.strip().splitlines() if ln.strip()]
    assert len(lines) == 1
    doc = json.loads(lines[0])
    assert doc["impl"] == "reference" and isinstance(doc["unavailable"], str) and "\n" not in doc["unavailable"]


def test_bench_help_lists_the_contract_flags():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True,
                       timeout=120, cwd=ROOT)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in r.stdout


def test_entry_module_has_build_and_smoke():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    assert callable(entry.build) and callable(entry.smoke)
