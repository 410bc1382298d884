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


def test_watchdog_restart_replaces_the_process_with_the_nccl_command_line(tmp_path):
    """The restart of a failed peer-transport run: the stalled process is replaced by the given command
    line, with the reason, a new rendezvous port and the agent store switched off in its environment."""
    child = tmp_path / "successor.py"
    child.write_text("import os, sys\n"
                     "print('ARGS', sys.argv[1:])\n"
                     "print('WHY', os.environ['MEGALODON_B200_BENCH_RESTARTED'])\n"
                     "print('PORT', os.environ['MASTER_PORT'], os.environ['TORCHELASTIC_USE_AGENT_STORE'])\n")
    driver = tmp_path / "driver.py"
    driver.write_text(
        "import importlib.util, os, sys, time\n"
        f"spec = importlib.util.spec_from_file_location('bench_module', {os.path.join(ROOT, 'bench.py')!r})\n"
        "bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)\n"
        "os.environ['MASTER_PORT'] = '29700'\n"
        f"dog = bench.StepWatchdog(3, 1.0, None, [{str(child)!r}, '--gpus', '4', '--transport', 'nccl'])\n"
        "dog.progress('warm-up step 0 done')\n"
        "time.sleep(30)\n"                     # the main thread "hangs"; the watchdog thread restarts the process
        "print('NOT REACHED')\n")
    out = subprocess.run([sys.executable, str(driver)], capture_output=True, text=True, cwd=ROOT, timeout=120)
    assert out.returncode == 0, out.stderr[-800:]
    assert "ARGS ['--gpus', '4', '--transport', 'nccl']" in out.stdout
    assert "WHY no step progress for 1 s (rank 3, after 'warm-up step 0 done')" in out.stdout
    assert "PORT 29701 False" in out.stdout
    assert "NOT REACHED" not in out.stdout
    assert "restarting with --transport nccl" in out.stderr
