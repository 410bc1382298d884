"""Parts of the benchmark contract that need no GPU."""
import dataclasses
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-500:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and "unavailable" in rec and "\n" not in rec["unavailable"]


def test_step_roofline_arithmetic():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from megalodon_b200.models.mega import ModelStore
    cfg = dataclasses.replace(ModelStore["mega7B_32k"])
    cfg.layerwise_ckpt, cfg.ckpt_layers = False, None
    plain = bench.step_roofline(cfg, 32768, 8, 350.0)
    cfg.layerwise_ckpt = True
    full = bench.step_roofline(cfg, 32768, 1, 3000.0)
    # 6 FLOPs per parameter and token without recomputation, 8 with: between 1.6 and 2.4 PFLOP per 32K step at 8.3 B
    assert 1.6 < plain["pflop_per_step"] < 1.9
    assert 2.2 < full["pflop_per_step"] < 2.5
    assert abs(full["pflop_per_step"] / plain["pflop_per_step"] - 4.0 / 3.0) < 0.03
    assert 0.0 < plain["fraction_of_sustained_cublas"] < 1.2
