"""Python host mirror of ``lve::WaterPhysics`` over the C ABI of include/neon_water.h.

Same shape as the engine's class (NeonEngine/src/water_physics.hpp:66-214): the constructor
takes the particle count's start positions and the uniform-block values and owns the device
buffers (water_physics.cpp:23-123); ``run_simulation`` records the passes of one or more steps
into a stream (``RunSimulation``, water_physics.cpp:131); positions are read back explicitly
(water_app.cpp:601-612).  Errors become ``RuntimeError``.  torch is optional and only
supplies streams; every kernel runs inside ``libneon_moe.so``.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .water_synth import WaterConfig


def make_config(cfg: WaterConfig, device: int = 0) -> "_lib.NeonWaterConfig":
    nx, ny, nz = cfg.grid_dim
    c = _lib.NeonWaterConfig(cfg.n_particles, nx, ny, nz, cfg.cell_size, cfg.over_relaxation, cfg.rest_density,
                             cfg.damping, cfg.mass, cfg.dt)
    c.box_min[:] = cfg.box_min
    c.box_max[:] = cfg.box_max
    c.gravity[:] = cfg.gravity
    c.collision_substeps, c.jacobi_iterations, c.device = cfg.collision_substeps, cfg.jacobi_iterations, device
    return c


class WaterPhysics:
    def __init__(self, cfg: WaterConfig, start_pos: np.ndarray, device: int = 0):
        self._lib = _lib.load()
        self.cfg = cfg
        self._c = make_config(cfg, device)
        start_pos = np.ascontiguousarray(start_pos, np.float32)
        assert start_pos.shape == (cfg.n_particles, 4)
        handle = ctypes.c_void_p()
        rc = self._lib.neon_water_create(ctypes.byref(self._c), ctypes.c_void_p(start_pos.ctypes.data), 0, ctypes.byref(handle))
        if rc != 0:
            raise RuntimeError(f"neon_water_create failed ({rc}): {self._lib.neon_water_last_error(None).decode()}")
        self._h = handle

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc}): {self._lib.neon_water_last_error(self._h).decode()}")

    def set_particles(self, pos4: np.ndarray, vel4: np.ndarray | None = None) -> None:
        pos4 = np.ascontiguousarray(pos4, np.float32)
        vel = None if vel4 is None else np.ascontiguousarray(vel4, np.float32)
        self._check(self._lib.neon_water_set_particles(self._h, ctypes.c_void_p(pos4.ctypes.data),
                                                       None if vel is None else ctypes.c_void_p(vel.ctypes.data), 0),
                    "neon_water_set_particles")

    def run_simulation(self, n_steps: int = 1, stream=None) -> None:
        st = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        self._check(self._lib.neon_water_step(self._h, int(n_steps), st), "neon_water_step")

    def run_host(self, pos4: np.ndarray, vel4: np.ndarray, n_steps: int = 1) -> None:
        """Host arrays in and out (updated in place)."""
        assert pos4.dtype == np.float32 and vel4.dtype == np.float32 and pos4.flags.c_contiguous and vel4.flags.c_contiguous
        self.run_host_ptr(pos4.ctypes.data, vel4.ctypes.data, n_steps)

    def run_host_ptr(self, pos_ptr: int, vel_ptr: int, n_steps: int = 1, stream=None) -> None:
        st = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        self._check(self._lib.neon_water_step_host(self._h, ctypes.c_void_p(pos_ptr), ctypes.c_void_p(vel_ptr), int(n_steps), st),
                    "neon_water_step_host")

    def read_particles(self):
        n = self.cfg.n_particles
        pos, vel = np.empty((n, 4), np.float32), np.empty((n, 4), np.float32)
        self._check(self._lib.neon_water_read_particles(self._h, ctypes.c_void_p(pos.ctypes.data), ctypes.c_void_p(vel.ctypes.data)),
                    "neon_water_read_particles")
        return pos, vel

    def read_grid(self, name: str) -> np.ndarray:
        out = np.empty(self.cfg.n_cells, np.uint32 if name == "flags" else np.float32)
        self._check(self._lib.neon_water_read_grid(self._h, name.encode(), ctypes.c_void_p(out.ctypes.data), out.nbytes),
                    "neon_water_read_grid")
        return out

    def read_grids(self) -> dict:
        return {k: self.read_grid(k) for k in ("u", "v", "w", "pressure", "density", "flags")}

    def device_pointers(self):
        p, v = ctypes.c_void_p(), ctypes.c_void_p()
        self._check(self._lib.neon_water_particles_device(self._h, ctypes.byref(p), ctypes.byref(v)), "neon_water_particles_device")
        return p.value, v.value

    def profile_step(self) -> dict:
        """One eager step timed in four groups (ms)."""
        ms = (ctypes.c_double * 4)()
        self._check(self._lib.neon_water_profile_step(self._h, ms, None), "neon_water_profile_step")
        return dict(zip(("separate", "particles_to_grid", "jacobi", "apply_g2p_integrate"), ms))

    def status(self) -> int:
        word = ctypes.c_int(0)
        self._lib.neon_water_status(self._h, ctypes.byref(word))
        return word.value

    def set_option(self, name: str, value: int) -> None:
        self._check(self._lib.neon_water_set_option(self._h, name.encode(), int(value)), "neon_water_set_option")

    def launch_count(self) -> int:
        return int(self._lib.neon_water_launch_count(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.neon_water_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
