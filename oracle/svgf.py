"""ctypes front end of the denoiser oracles (temporal accumulation + a-trous filter).

TEST INFRASTRUCTURE ONLY (tests/, smoke check, CPU-baseline leg of the benchmark).

* :func:`frame` runs oracle/svgf_oracle.c, the restatement (always available: gcc builds it).
* :func:`ref_frame` runs oracle/_ref/libsvgf_ref.so, the reference engine's own two shaders
  compiled for the CPU by oracle/svgf_ref_build.py (present where the reference checkout was
  available when the library was built; it travels as a built file).
Both work in place on a :class:`State` and a frame's rgba8 image.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
SO = os.path.join(BUILD_DIR, "libsvgf_oracle.so")
SRC = os.path.join(HERE, "svgf_oracle.c")
REF_SO = os.path.join(HERE, "_ref", "libsvgf_ref.so")


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
        _lib.svgf_oracle_frame.restype = ctypes.c_int
        _lib.svgf_oracle_exp2.restype = ctypes.c_float
        _lib.svgf_oracle_exp2.argtypes = [ctypes.c_float]
    return _lib


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(REF_SO)
        _ref.svgf_ref_frame.restype = ctypes.c_int
    return _ref


@dataclass
class State:
    """What the denoiser keeps between frames: the two rgba16f history images (raw half bits),
    the rgba32f moments image and the ping-pong flag (RayTracingRast::pingPong, initially false)."""
    colour_a: np.ndarray
    colour_b: np.ndarray
    data: np.ndarray
    ping_pong: int = 0

    @classmethod
    def zeros(cls, w: int, h: int) -> "State":
        return cls(np.zeros((h, w, 4), np.uint16), np.zeros((h, w, 4), np.uint16), np.zeros((h, w, 4), np.float32), 0)

    def copy(self) -> "State":
        return State(self.colour_a.copy(), self.colour_b.copy(), self.data.copy(), self.ping_pong)


def _run(fn, gbuffer, image: np.ndarray, st: State, atrous_iterations: int, last: int):
    h, w = image.shape[:2]
    for a, dt in list(zip(gbuffer, (np.float32,) * 4)) + [(image, np.uint8), (st.colour_a, np.uint16), (st.colour_b, np.uint16),
                                                          (st.data, np.float32)]:
        assert a.dtype == dt and a.shape == (h, w, 4) and a.flags.c_contiguous
    vp = lambda a: ctypes.c_void_p(a.ctypes.data)  # noqa: E731
    pp = ctypes.c_int(st.ping_pong)
    rc = fn(ctypes.c_int(w), ctypes.c_int(h), *(vp(a) for a in gbuffer), vp(image), vp(st.colour_a), vp(st.colour_b), vp(st.data),
            ctypes.byref(pp), ctypes.c_int(atrous_iterations), ctypes.c_int(last))
    if rc:
        raise RuntimeError(f"denoiser frame failed ({rc})")
    st.ping_pong = pp.value


def frame(gbuffer, image: np.ndarray, st: State, atrous_iterations: int = 3, serial: bool = False):
    """Restatement.  gbuffer = (position, normal, barycentric, motion), each float32 [h, w, 4].
    serial=True: in-place moments in ascending pixel order (the serially executed reference);
    serial=False: every pass reads the moments of the previous pass (what the CUDA kernels do)."""
    _run(lib().svgf_oracle_frame, gbuffer, image, st, atrous_iterations, int(serial))


def ref_frame(gbuffer, image: np.ndarray, st: State, atrous_iterations: int = 3, honour_early_return: bool = False):
    """The reference shaders themselves, executed serially on the CPU.  honour_early_return=True
    keeps the `return;` both shaders start with in the checkout (every pass then does nothing)."""
    _run(ref_lib().svgf_ref_frame, gbuffer, image, st, atrous_iterations, int(honour_early_return))


def exp2(x: float) -> float:
    return float(lib().svgf_oracle_exp2(ctypes.c_float(x)))
