"""The benchmark's reference arm needs no GPU: its JSON line must keep the contract, and it must not pull the product
library into the process (the arm times the CPU restatement, nothing of the CUDA path)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_line_and_isolation():
    code = (
        "import sys, json, types\n"
        "sys.argv = ['bench.py', '--impl', 'reference', '--steps', '1', '--warmup', '0']\n"
        "import runpy\n"
        "runpy.run_path('bench.py', run_name='__main__')\n"
        "maps = open('/proc/self/maps').read()\n"
        "print('LIBMIE_MAPPED', 'libmie.so' in maps)\n"
        "print('PACKAGE_NATIVE_IMPORTED', 'maskedincrementeval_b200._native' in sys.modules)\n"
    )
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    line = json.loads(next(ln for ln in lines if ln.startswith("{")))
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["value"] > 0
    assert line["config"]["workload"] == "e2depth_260x346_b1"
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "LIBMIE_MAPPED False" in r.stdout and "PACKAGE_NATIVE_IMPORTED False" in r.stdout
