"""Python mirror of an engine-style `lve::PathTracerSystem` over the C ABI in include/neon_pt.h: the
constructor takes the flattened scene (as `RayTracingSystem` takes vertices, indices, materials and
light positions, NeonEngine/src/raytracing_system.cpp:19-68), `render` records one frame into a
stream, a non-zero status becomes a RuntimeError.  torch only owns device memory and streams."""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .pt_synth import MATERIAL_DTYPE, VERTEX_DTYPE, PtScene


class PathTracer:
    def __init__(self, scene: PtScene, width: int = 800, height: int = 600, device: int = 0):
        self._lib = _lib.load()
        self.width, self.height, self.device = int(width), int(height), int(device)
        v = np.ascontiguousarray(scene.vertices, VERTEX_DTYPE)
        i = np.ascontiguousarray(scene.indices, np.uint32)
        m = np.ascontiguousarray(scene.materials, MATERIAL_DTYPE)
        cfg = _lib.NeonPtConfig(self.width, self.height, int(scene.n_lights), self.device)
        h = ctypes.c_void_p()
        rc = self._lib.neon_pt_create(ctypes.byref(cfg), v.ctypes.data, len(v), i.ctypes.data, len(i), m.ctypes.data, len(m), ctypes.byref(h))
        if rc != 0:
            raise RuntimeError(f"neon_pt_create failed ({rc}): {self._lib.neon_pt_last_error(None).decode()}")
        self._h = h

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc}): {self._lib.neon_pt_last_error(self._h).decode()}")

    @staticmethod
    def _mat(a):
        a = np.ascontiguousarray(a, np.float32)
        assert a.size == 16
        return a

    def render(self, inverse_projection, inverse_view, frame_id: float, image=None, stream=None):
        """One frame into a torch uint8 [height, width, 4] tensor on this tracer's GPU."""
        import torch
        if image is None:
            image = torch.empty((self.height, self.width, 4), dtype=torch.uint8, device=f"cuda:{self.device}")
        ip, iv = self._mat(inverse_projection), self._mat(inverse_view)
        st = (stream or torch.cuda.current_stream(image.device)).cuda_stream
        self._check(self._lib.neon_pt_render(self._h, ip.ctypes.data, iv.ctypes.data, ctypes.c_float(frame_id), image.data_ptr(), st), "neon_pt_render")
        return image

    def render_host(self, inverse_projection, inverse_view, frame_id: float) -> np.ndarray:
        out = np.empty((self.height, self.width, 4), np.uint8)
        ip, iv = self._mat(inverse_projection), self._mat(inverse_view)
        self._check(self._lib.neon_pt_render_host(self._h, ip.ctypes.data, iv.ctypes.data, ctypes.c_float(frame_id), out.ctypes.data), "neon_pt_render_host")
        return out

    def render_host_ptr(self, ip, iv, frame_id: float, out_ptr: int) -> None:
        self._check(self._lib.neon_pt_render_host(self._h, ip.ctypes.data, iv.ctypes.data, ctypes.c_float(frame_id), out_ptr), "neon_pt_render_host")

    def rays(self) -> int:
        n = ctypes.c_uint64(0)
        self._check(self._lib.neon_pt_rays(self._h, ctypes.byref(n)), "neon_pt_rays")
        return n.value

    def bvh_info(self):
        a, b = ctypes.c_int(0), ctypes.c_int(0)
        self._lib.neon_pt_bvh_info(self._h, ctypes.byref(a), ctypes.byref(b))
        return a.value, b.value

    def status(self) -> int:
        w = ctypes.c_int(0)
        self._lib.neon_pt_status(self._h, ctypes.byref(w))
        return w.value

    def launch_count(self) -> int:
        return int(self._lib.neon_pt_launch_count(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.neon_pt_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
