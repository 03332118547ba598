"""The headless engine-style application loop (neonengine_b200/csrc/moe_app.cpp): runs frames of
the layer for a second, prints throughput the way the engine's apps print FPS, exits 0."""
import os
import re
import subprocess

import pytest

from neonengine_b200 import build, synth, weight_file

pytestmark = pytest.mark.gpu


def _run(args):
    build.build()
    assert os.path.exists(build.APP)
    return subprocess.run([build.APP, *args], capture_output=True, text=True, timeout=300)


def test_app_loop_reports_tokens_per_second():
    res = _run(["--hidden", "256", "--inter", "192", "--experts", "8", "--tokens", "16", "--seconds", "1.3"])
    assert res.returncode == 0, res.stderr
    m = re.search(r"MoE layer \| tokens/s: ([0-9.]+) \(([0-9.]+) ms per pass of 16 tokens\)", res.stdout)
    assert m and float(m.group(1)) > 1000.0, res.stdout
    assert "device status: 0" in res.stdout


def test_app_loads_a_weight_file(tmp_path):
    shape = synth.MoeShape(hidden=256, inter=192, n_experts=8, top_k=4)
    path = str(tmp_path / "layer.nmoe")
    weight_file.write_raw(path, synth.make_weights(shape, 1))
    res = _run(["--weights", path, "--hidden", "256", "--inter", "192", "--experts", "8", "--tokens", "4", "--seconds", "0.3"])
    assert res.returncode == 0 and "device status: 0" in res.stdout, res.stdout + res.stderr
    bad = _run(["--weights", path, "--hidden", "256", "--inter", "128", "--experts", "8", "--tokens", "4", "--seconds", "0.2"])
    assert bad.returncode == 1 and "expects" in bad.stderr
