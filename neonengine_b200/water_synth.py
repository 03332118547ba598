"""Parameters and seeded particle spawn of the reference engine's water demo.

Values follow NeonEngine/src/water_app.cpp: 20^3 = 8000 particles (:59-61), box
(-4.928, -3.08, -1.848)..(4.928, 0.55, 2.464) (:150-151), cell size 0.1 and the grid that covers
the box, 99 x 37 x 44 (:172-185), over-relaxation 1.03, rest density 1, gravity (0, 98.1, 0),
FLIP ratio 0, particle mass 20 (:243-255), time step 1/500, 4 separation sub-steps and 50 Jacobi
iterations per step (NeonEngine/src/water_physics.cpp:211, :243, :321).  The spawn restates
:260-306: a regular lattice inside 0.9 x box minus one cell, jittered by a Mersenne twister
seeded with 42 (uniform in +-0.5 x 0.396, three draws per particle in x, y, z order; the draw is
raw / 2^32 in 32-bit floats, as libstdc++'s uniform_real_distribution<float> forms it).
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np


@dataclasses.dataclass
class WaterConfig:
    particles_per_side: int = 20
    box_min: tuple = (-4.928, -3.08, -1.848)
    box_max: tuple = (4.928, 0.55, 4.928 / 2.0)
    cell_size: float = 0.1
    over_relaxation: float = 1.03
    rest_density: float = 1.0
    damping: float = 0.0          # FLIP ratio (0 = pure PIC, as the app sets it)
    mass: float = 20.0
    dt: float = 1.0 / 500.0
    gravity: tuple = (0.0, 9.81 * 10.0, 0.0)
    collision_substeps: int = 4
    jacobi_iterations: int = 50

    @property
    def n_particles(self) -> int:
        return self.particles_per_side ** 3

    @property
    def grid_dim(self) -> tuple:
        f = np.float32
        size = [f(self.box_max[a]) - f(self.box_min[a]) for a in range(3)]
        return tuple(max(int(math.ceil(float(s / f(self.cell_size)))), 2) for s in size)

    @property
    def n_cells(self) -> int:
        nx, ny, nz = self.grid_dim
        return nx * ny * nz


def spawn_particles(cfg: WaterConfig, seed: int = 42) -> np.ndarray:
    """float32 [N, 4] positions (w = 1, as the engine uploads them)."""
    f = np.float32
    L = cfg.particles_per_side
    bit = np.random.MT19937()
    bit._legacy_seeding(seed)  # init_genrand(seed), the seeding std::mt19937(seed) uses
    raw = bit.random_raw(3 * L ** 3).astype(np.float32)
    r = raw / f(4294967296.0)
    r = np.where(r >= f(1.0), np.nextafter(f(1.0), f(0.0)), r).astype(np.float32)
    jitter = (r * f(1.0) + f(-0.5)).astype(np.float32).reshape(-1, 3)
    particle_scale = f(0.2)
    spacing = f(2.2) * particle_scale
    jitter_scale = spacing * f(0.9)
    bmin = np.array(cfg.box_min, np.float32) * f(0.9)
    bmax = np.array(cfg.box_max, np.float32) * f(0.9)
    margin = f(cfg.cell_size)
    smin, smax = bmin + margin, bmax - margin
    size = smax - smin
    eps = f(0.001)
    pos = np.zeros((L ** 3, 4), np.float32)
    draw = 0
    for x in range(L):
        for y in range(L):
            for z in range(L):
                n = [(f(c) + eps) / (f(L - 1) + f(2.0) * eps) if L > 1 else f(0.5) for c in (x, y, z)]
                p = smin + np.array(n, np.float32) * size
                p = p + jitter[draw] * jitter_scale
                draw += 1
                pos[x + y * L + z * L * L, :3] = p
    pos[:, 3] = 1.0
    return pos
