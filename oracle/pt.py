"""ctypes front end of the path-tracer oracles: the reference engine's own shaders compiled for the CPU
(oracle/_ref/libpt_ref.so, built by pt_ref_build.py where the reference checkout is present) and the
plain-C restatement (pt_oracle.c).  Test infrastructure: only tests, the smoke check and the benchmark's
CPU leg import this module."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "pt_oracle.c")
_SO = os.path.join(_HERE, "_build", "libpt_oracle.so")
_lib = None
_ref = None


def build(force: bool = False) -> str:
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    os.makedirs(os.path.dirname(_SO), exist_ok=True)
    subprocess.run(["gcc", "-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fPIC", "-shared", "-std=c11", _SRC, "-o", _SO, "-lm"],
                   check=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.pt_oracle_render.restype = ctypes.c_ulonglong
    return _lib


def have_ref() -> bool:
    from . import pt_ref_build
    return pt_ref_build.build() is not None


def ref_lib() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        from . import pt_ref_build
        so = pt_ref_build.build()
        if so is None:
            raise RuntimeError("the compiled reference shaders are not available here")
        _ref = ctypes.CDLL(so)
        _ref.pt_ref_render.restype = ctypes.c_ulonglong
    return _ref


def _render(fn, scene, inv_proj, inv_view, frame_id, width, height):
    v = np.ascontiguousarray(scene.vertices)
    i = np.ascontiguousarray(scene.indices, np.uint32)
    m = np.ascontiguousarray(scene.materials)
    ip = np.ascontiguousarray(inv_proj, np.float32)
    iv = np.ascontiguousarray(inv_view, np.float32)
    img = np.zeros((height, width, 4), np.uint8)
    rays = fn(ctypes.c_void_p(v.ctypes.data), len(v), ctypes.c_void_p(i.ctypes.data), len(i), ctypes.c_void_p(m.ctypes.data), len(m),
              int(scene.n_lights), ctypes.c_void_p(ip.ctypes.data), ctypes.c_void_p(iv.ctypes.data), ctypes.c_float(frame_id),
              int(width), int(height), ctypes.c_void_p(img.ctypes.data))
    return img, int(rays)


def ref_render(scene, inv_proj, inv_view, frame_id, width, height):
    """One frame by the reference's own shaders compiled for the CPU: (rgba8 image, rays traced)."""
    return _render(ref_lib().pt_ref_render, scene, inv_proj, inv_view, frame_id, width, height)


def render(scene, inv_proj, inv_view, frame_id, width, height):
    """One frame by the C restatement: (rgba8 image, rays traced)."""
    return _render(lib().pt_oracle_render, scene, inv_proj, inv_view, frame_id, width, height)
