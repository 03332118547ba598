"""CPU tests of the FLIP water-step restatement (oracle/water_oracle.c): pinned bit for bit
against the fixture the reference engine's own shader produced (tests/golden/water_small.npz,
made by tests/golden/make_water_golden.py) and, where the compiled reference shader is present
(oracle/_ref/libwater_ref.so), against it directly at the demo's full size."""
import dataclasses
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))

from make_water_golden import oracle_params, small_config  # noqa: E402
from neonengine_b200.water_synth import WaterConfig, spawn_particles  # noqa: E402
from oracle import water  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "water_small.npz")


def test_demo_configuration():
    cfg = WaterConfig()
    assert cfg.n_particles == 8000 and cfg.grid_dim == (99, 37, 44) and cfg.n_cells == 161172
    pos = spawn_particles(cfg)
    assert pos.shape == (8000, 4) and pos.dtype == np.float32 and (pos[:, 3] == 1.0).all()
    np.testing.assert_array_equal(pos, spawn_particles(cfg))
    assert len(np.unique(pos[:, :3], axis=0)) == 8000


def test_restatement_reproduces_reference_fixture_bit_for_bit():
    z = np.load(GOLDEN)
    cfg = small_config()
    np.testing.assert_array_equal(spawn_particles(cfg), z["pos0"])
    pos, vel = z["pos0"].copy(), np.zeros_like(z["pos0"])
    for step in (1, 2, 3):
        grids = water.step(oracle_params(cfg), pos, vel, 1, collision_mode=0)
        np.testing.assert_array_equal(pos, z[f"pos{step}"])
        np.testing.assert_array_equal(vel, z[f"vel{step}"])
    for k, v in grids.items():
        np.testing.assert_array_equal(v, z["grid_" + k], err_msg=k)
    # several steps in one call equal single-step calls
    pos2, vel2 = z["pos0"].copy(), np.zeros_like(z["pos0"])
    water.step(oracle_params(cfg), pos2, vel2, 3, collision_mode=0)
    np.testing.assert_array_equal(pos2, z["pos3"])


@pytest.mark.skipif(not water.have_ref(), reason="compiled reference shader not present")
def test_restatement_equals_compiled_reference_shader_at_demo_size():
    cfg = WaterConfig()
    pos0 = spawn_particles(cfg)
    a, va = pos0.copy(), np.zeros_like(pos0)
    b, vb = pos0.copy(), np.zeros_like(pos0)
    ga = water.step(oracle_params(cfg), a, va, 2, collision_mode=0)
    gb = water.ref_step(oracle_params(cfg), b, vb, 2)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(va, vb)
    for k in ga:
        np.testing.assert_array_equal(ga[k], gb[k], err_msg=k)


def test_modes_agree_without_separation_and_edge_cases():
    cfg = dataclasses.replace(small_config(), collision_substeps=0)
    pos0 = spawn_particles(cfg)
    a, va = pos0.copy(), np.zeros_like(pos0)
    b, vb = pos0.copy(), np.zeros_like(pos0)
    water.step(oracle_params(cfg), a, va, 2, collision_mode=0)
    water.step(oracle_params(cfg), b, vb, 2, collision_mode=1)
    np.testing.assert_array_equal(a, b)
    # no pressure iterations, a single particle: gravity and the wall clamp still apply
    cfg1 = dataclasses.replace(small_config(), particles_per_side=1, jacobi_iterations=0)
    p = spawn_particles(cfg1)
    v = np.zeros_like(p)
    y0 = p[0, 1]
    g = water.step(oracle_params(cfg1), p, v, 1)
    assert v[0, 1] > 0 and p[0, 1] > y0 and p[0, 3] == np.float32(0.1)
    assert (g["pressure"] == 0).all() and int((g["flags"] & 1).sum()) > 0


def test_particles_stay_inside_the_walls():
    cfg = small_config()
    pos, vel = spawn_particles(cfg), None
    vel = np.zeros_like(pos)
    water.step(oracle_params(cfg), pos, vel, 20, collision_mode=1)
    lo = np.array(cfg.box_min, np.float32) + np.float32(cfg.cell_size)
    hi = np.array(cfg.box_max, np.float32) - np.float32(cfg.cell_size)
    assert (pos[:, :3] >= lo).all() and (pos[:, :3] <= hi).all() and np.isfinite(vel).all()
