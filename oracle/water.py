"""ctypes front end of the FLIP water-step oracles.

TEST INFRASTRUCTURE ONLY (tests/, smoke check, CPU-baseline leg of the benchmark).

* :func:`step` runs oracle/water_oracle.c, the restatement (always available: gcc builds it).
* :func:`ref_step` runs oracle/_ref/libwater_ref.so, the reference engine's own shader compiled
  for the CPU by oracle/water_ref_build.py (present where the reference checkout was available
  when the library was built; it travels as a built file).
Both advance positions/velocities in place and return the grids of the last step.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
SO = os.path.join(BUILD_DIR, "libwater_oracle.so")
SRC = os.path.join(HERE, "water_oracle.c")
REF_SO = os.path.join(HERE, "_ref", "libwater_ref.so")


class WaterParams(ctypes.Structure):
    """Mirror of `water_params` (water_oracle.c) / `water_ref_params` / `neon_water_config`'s physics part."""
    _fields_ = [("n_particles", ctypes.c_int), ("nx", ctypes.c_int), ("ny", ctypes.c_int), ("nz", ctypes.c_int),
                ("cell_size", ctypes.c_float), ("over_relaxation", ctypes.c_float), ("rest_density", ctypes.c_float),
                ("damping", ctypes.c_float), ("mass", ctypes.c_float), ("dt", ctypes.c_float),
                ("box_min", ctypes.c_float * 3), ("box_max", ctypes.c_float * 3), ("gravity", ctypes.c_float * 3),
                ("collision_substeps", ctypes.c_int), ("jacobi_iterations", ctypes.c_int)]


def build(force: bool = False) -> str:
    if not force and os.path.exists(SO) and os.path.getmtime(SO) >= os.path.getmtime(SRC):
        return SO
    os.makedirs(BUILD_DIR, exist_ok=True)
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-std=c11", "-shared", "-fPIC", SRC, "-o", SO, "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError("gcc failed: " + res.stderr)
    return SO


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.water_oracle_step.restype = ctypes.c_int
    return _lib


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(REF_SO)
        _ref.water_ref_step.restype = ctypes.c_int
    return _ref


def _run(fn, params: WaterParams, pos4: np.ndarray, vel4: np.ndarray, n_steps: int, extra):
    assert pos4.dtype == np.float32 and vel4.dtype == np.float32 and pos4.flags.c_contiguous and vel4.flags.c_contiguous
    assert pos4.shape == (params.n_particles, 4) and vel4.shape == pos4.shape
    C = params.nx * params.ny * params.nz
    out = {k: np.empty(C, np.float32) for k in ("u", "v", "w", "pressure", "density")}
    out["flags"] = np.empty(C, np.uint32)
    vp = lambda a: ctypes.c_void_p(a.ctypes.data)  # noqa: E731
    rc = fn(ctypes.byref(params), vp(pos4), vp(vel4), ctypes.c_int(n_steps), *extra, vp(out["u"]), vp(out["v"]), vp(out["w"]),
            vp(out["pressure"]), vp(out["flags"]), vp(out["density"]))
    if rc:
        raise RuntimeError(f"water step failed ({rc})")
    return out


def step(params: WaterParams, pos4: np.ndarray, vel4: np.ndarray, n_steps: int = 1, collision_mode: int = 1):
    """Restatement.  collision_mode 0 = serial in-place separation pass (the serially executed
    reference), 1 = separation pass on a snapshot (what a parallel implementation reproduces)."""
    return _run(lib().water_oracle_step, params, pos4, vel4, n_steps, (ctypes.c_int(collision_mode),))


def ref_step(params: WaterParams, pos4: np.ndarray, vel4: np.ndarray, n_steps: int = 1):
    """The reference shader itself, executed serially on the CPU."""
    return _run(ref_lib().water_ref_step, params, pos4, vel4, n_steps, ())
