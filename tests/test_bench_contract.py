"""CPU checks of bench.py's contract: the reference arm prints exactly one JSON line on stdout with
the agreed keys, for the MoE layer (CPU oracle) and for the water step and the denoiser (the reference shaders
compiled for the CPU when present, else the restatements)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"}


def _run(args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *args],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, res.stdout
    return json.loads(lines[0])


def test_reference_arm_water():
    line = _run(["--workload", "water", "--steps", "1"])
    assert KEYS <= set(line) and line["impl"] == "reference" and line["metric"] == "water_steps_per_s"
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] == 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert line["config"]["workload"] == "water"


def test_reference_arm_denoiser():
    line = _run(["--workload", "svgf", "--steps", "1"])
    assert KEYS <= set(line) and line["impl"] == "reference" and line["metric"] == "denoised_frames_per_s"
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] == 1
    assert line["e2e"]["value"] == line["value"] and line["config"]["workload"] == "svgf"


def test_reference_arm_moe_layer_under_torchrun_env():
    """Rank 0 prints the line; any other rank prints nothing and exits 0."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
