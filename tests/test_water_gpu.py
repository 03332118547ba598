"""GPU parity of the FLIP water step (include/neon_water.h) against the restatement of the
reference shader (oracle/water_oracle.c, itself pinned to the compiled shader).  Bit-exact:
the kernels use the shader's float operations in the shader's order (no fused multiply-add),
the separation pass is compared in the snapshot form (collision_mode 1), and without
separation sub-steps the result must equal the serially executed reference as well."""
import dataclasses
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))

pytestmark = pytest.mark.gpu

from make_water_golden import oracle_params, small_config  # noqa: E402
from neonengine_b200.water_synth import WaterConfig, spawn_particles  # noqa: E402
from oracle import water  # noqa: E402


def _gpu(cfg, pos0):
    from neonengine_b200.water_physics import WaterPhysics
    return WaterPhysics(cfg, pos0)


def _compare(sim, pos, vel, grids):
    assert sim.status() == 0
    gp, gv = sim.read_particles()
    np.testing.assert_array_equal(gp, pos)
    np.testing.assert_array_equal(gv, vel)
    got = sim.read_grids()
    for k in grids:
        np.testing.assert_array_equal(got[k], grids[k], err_msg=k)


@pytest.mark.parametrize("steps", [1, 3])
def test_small_case_bit_exact(steps):
    cfg = small_config()
    pos0 = spawn_particles(cfg)
    sim = _gpu(cfg, pos0)
    sim.run_simulation(steps)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    grids = water.step(oracle_params(cfg), pos, vel, steps, collision_mode=1)
    _compare(sim, pos, vel, grids)
    sim.close()


def test_demo_size_bit_exact():
    cfg = WaterConfig()
    pos0 = spawn_particles(cfg)
    sim = _gpu(cfg, pos0)
    sim.run_simulation(2)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    grids = water.step(oracle_params(cfg), pos, vel, 2, collision_mode=1)
    _compare(sim, pos, vel, grids)
    assert int((grids["flags"] & 1).sum()) > 50000
    sim.close()


def test_without_separation_equals_the_serial_reference():
    """No separation sub-steps: every remaining pass is order-independent once the grid sums add
    in particle order, so the kernels must equal the fixture's producer (mode 0) exactly; with
    the compiled reference shader present, compare against it directly."""
    cfg = dataclasses.replace(small_config(), collision_substeps=0)
    pos0 = spawn_particles(cfg)
    sim = _gpu(cfg, pos0)
    sim.run_simulation(3)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    run = water.ref_step if water.have_ref() else (lambda p, a, b, n: water.step(p, a, b, n, collision_mode=0))
    grids = run(oracle_params(cfg), pos, vel, 3)
    _compare(sim, pos, vel, grids)
    sim.close()


def test_graph_eager_host_paths_and_determinism():
    cfg = small_config()
    pos0 = spawn_particles(cfg)
    a = _gpu(cfg, pos0)
    a.run_simulation(4)
    pa, va = a.read_particles()
    b = _gpu(cfg, pos0)
    b.set_option("use_graphs", 0)
    for _ in range(4):
        b.run_simulation(1)
    pb, vb = b.read_particles()
    np.testing.assert_array_equal(pa, pb)
    np.testing.assert_array_equal(va, vb)
    ph, vh = pos0.copy(), np.zeros_like(pos0)
    b.run_host(ph, vh, 4)
    np.testing.assert_array_equal(ph, pa)
    np.testing.assert_array_equal(vh, va)
    before = a.launch_count()
    a.set_particles(pos0)
    a.run_simulation(4)
    assert a.launch_count() > before
    np.testing.assert_array_equal(a.read_particles()[0], pa)
    p_dev, v_dev = a.device_pointers()
    assert p_dev and v_dev
    a.close()
    b.close()


def test_odd_substeps_and_no_jacobi():
    cfg = dataclasses.replace(small_config(), collision_substeps=3, jacobi_iterations=0)
    pos0 = spawn_particles(cfg)
    sim = _gpu(cfg, pos0)
    sim.run_simulation(2)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    grids = water.step(oracle_params(cfg), pos, vel, 2, collision_mode=1)
    _compare(sim, pos, vel, grids)
    cfg = dataclasses.replace(small_config(), jacobi_iterations=7)
    sim2 = _gpu(cfg, pos0)
    sim2.run_simulation(1)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    grids = water.step(oracle_params(cfg), pos, vel, 1, collision_mode=1)
    _compare(sim2, pos, vel, grids)
    sim.close()
    sim2.close()


def test_fused_and_per_iteration_jacobi_agree():
    cfg = WaterConfig()
    pos0 = spawn_particles(cfg)
    outs = []
    for fused in (1, 0):
        sim = _gpu(cfg, pos0)
        sim.set_option("fused_jacobi", fused)
        sim.run_simulation(3)
        assert sim.status() == 0
        outs.append((sim.read_particles(), sim.read_grid("pressure")))
        sim.close()
    np.testing.assert_array_equal(outs[0][0][0], outs[1][0][0])
    np.testing.assert_array_equal(outs[0][0][1], outs[1][0][1])
    np.testing.assert_array_equal(outs[0][1], outs[1][1])


def test_rejects_bad_arguments():
    cfg = small_config()
    sim = _gpu(cfg, spawn_particles(cfg))
    with pytest.raises(RuntimeError):
        sim.run_simulation(-1)
    with pytest.raises(RuntimeError):
        sim.set_option("nonsense", 1)
    with pytest.raises(RuntimeError, match="unknown grid"):
        sim.read_grid("vorticity")
    sim.close()


def test_fine_grid_beyond_the_fused_kernel_limit():
    """Half the cell size: 1.25 M cells, more than the cooperative Jacobi kernel covers (two cells
    per resident thread), so the step falls back to one launch per iteration, and the prefix sum
    runs over more than 1024 blocks.  Still bit-exact."""
    cfg = dataclasses.replace(WaterConfig(), cell_size=0.05, jacobi_iterations=12)
    assert cfg.n_cells > 2 * 148 * 1024
    pos0 = spawn_particles(cfg)
    sim = _gpu(cfg, pos0)
    sim.run_simulation(2)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    grids = water.step(oracle_params(cfg), pos, vel, 2, collision_mode=1)
    _compare(sim, pos, vel, grids)
    sim.close()


def test_more_particles_than_the_demo():
    """27 000 particles (30^3) in the demo box: groups, boxes and bins at a larger size."""
    cfg = dataclasses.replace(WaterConfig(), particles_per_side=30, jacobi_iterations=10, collision_substeps=2)
    pos0 = spawn_particles(cfg)
    sim = _gpu(cfg, pos0)
    sim.run_simulation(1)
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    grids = water.step(oracle_params(cfg), pos, vel, 1, collision_mode=1)
    _compare(sim, pos, vel, grids)
    sim.close()
