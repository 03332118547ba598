"""Generates tests/golden/water_small.npz from the reference engine's own water shader compiled
for the CPU (oracle/water_ref_build.py -> oracle/_ref/libwater_ref.so; needs the reference
checkout).  Small case so the fixture stays a few tens of KB: 6^3 = 216 particles in a
21 x 13 x 15-cell box, the app's physical constants, 3 steps.

    python tests/golden/make_water_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from neonengine_b200.water_synth import WaterConfig, spawn_particles  # noqa: E402
from oracle import water, water_ref_build  # noqa: E402


def small_config() -> WaterConfig:
    return WaterConfig(particles_per_side=6, box_min=(-1.0, -0.8, -0.7), box_max=(1.1, 0.45, 0.8))


def oracle_params(cfg: WaterConfig) -> "water.WaterParams":
    nx, ny, nz = cfg.grid_dim
    p = water.WaterParams(cfg.n_particles, nx, ny, nz, cfg.cell_size, cfg.over_relaxation, cfg.rest_density, cfg.damping,
                          cfg.mass, cfg.dt)
    p.box_min[:] = cfg.box_min
    p.box_max[:] = cfg.box_max
    p.gravity[:] = cfg.gravity
    p.collision_substeps, p.jacobi_iterations = cfg.collision_substeps, cfg.jacobi_iterations
    return p


if __name__ == "__main__":
    if water_ref_build.build(force=True) is None:
        raise SystemExit("the reference checkout is not available: cannot regenerate the fixture")
    cfg = small_config()
    pos0 = spawn_particles(cfg)
    out = {"pos0": pos0}
    pos, vel = pos0.copy(), np.zeros_like(pos0)
    for step in (1, 2, 3):
        grids = water.ref_step(oracle_params(cfg), pos, vel, 1)
        out[f"pos{step}"], out[f"vel{step}"] = pos.copy(), vel.copy()
    for k, v in grids.items():
        out["grid_" + k] = v
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "water_small.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes; grid", cfg.grid_dim, "fluid cells", int((grids["flags"] & 1).sum()))
