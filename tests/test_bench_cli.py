"""bench.py on a machine without a GPU: the parts of its contract that need no device."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_operator_sweep_has_no_reference_arm():
    line = _run("--impl", "reference", "--config", "2")
    assert line["impl"] == "reference" and "unavailable" in line


def test_every_configuration_is_selectable():
    sys.path.insert(0, ROOT)
    import bench
    assert sorted(bench.CONFIGS) == [1, 2, 3, 4, 5]
    for n, c in bench.CONFIGS.items():
        bench.select_config(n)
        assert bench.WORKLOAD == c["workload"] and bench.N_CTX == c["n_ctx"]
    bench.select_config(1)
    peak, kind = bench.measured_peak()
    assert peak > 1000 and kind in ("measured", "fallback")
    assert bench.bf16_peak_tflops() > 100
