"""Python host mirror of the denoiser part of ``lve::RayTracingRast`` over the C ABI of
include/neon_svgf.h.

Same shape as the engine's class: the constructor owns the history images
(NeonEngine/src/raytracing_rast.cpp:120-160), ``render`` records the temporal pass and the
a-trous passes of one frame into a stream (``renderCompute`` + ``renderAtrous``,
raytracing_rast.cpp:325-428, called as raytracing_app.cpp:735-765), the state is read back
explicitly.  Errors become ``RuntimeError``.  torch is optional and only supplies streams and
device buffers; every kernel runs inside ``libneon_moe.so``.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib


class SvgfDenoiser:
    def __init__(self, width: int, height: int, atrous_iterations: int = 3, device: int = 0):
        self._lib = _lib.load()
        self.width, self.height, self.atrous_iterations = width, height, atrous_iterations
        cfg = _lib.NeonSvgfConfig(width, height, atrous_iterations, device)
        handle = ctypes.c_void_p()
        rc = self._lib.neon_svgf_create(ctypes.byref(cfg), ctypes.byref(handle))
        if rc != 0:
            raise RuntimeError(f"neon_svgf_create failed ({rc}): {self._lib.neon_svgf_last_error(None).decode()}")
        self._h = handle

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc}): {self._lib.neon_svgf_last_error(self._h).decode()}")

    def set_history(self, colour_a=None, colour_b=None, moments=None, ping_pong: int = 0) -> None:
        """Host arrays (uint16 / uint16 / float32, each [h, w, 4]) or None = zeros."""
        keep = [None if a is None else np.ascontiguousarray(a, dt) for a, dt in
                ((colour_a, np.uint16), (colour_b, np.uint16), (moments, np.float32))]
        ptr = [None if a is None else ctypes.c_void_p(a.ctypes.data) for a in keep]
        self._check(self._lib.neon_svgf_set_history(self._h, *ptr, int(ping_pong), 0), "neon_svgf_set_history")

    def render_ptr(self, position: int, normal: int, barycentric: int, motion: int, image: int, stream=None) -> None:
        """Device addresses; asynchronous."""
        st = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        self._check(self._lib.neon_svgf_denoise(self._h, *(ctypes.c_void_p(p) for p in (position, normal, barycentric, motion, image)),
                                                st), "neon_svgf_denoise")

    def render(self, gbuffer, image, stream=None) -> None:
        """gbuffer = four torch float32 CUDA tensors [h, w, 4]; image = torch uint8 CUDA tensor [h, w, 4] (in place)."""
        self.render_ptr(*(t.data_ptr() for t in gbuffer), image.data_ptr(), stream)

    def render_host_ptr(self, position: int, normal: int, barycentric: int, motion: int, image: int, stream=None) -> None:
        st = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        self._check(self._lib.neon_svgf_denoise_host(self._h, *(ctypes.c_void_p(p) for p in (position, normal, barycentric, motion, image)),
                                                     st), "neon_svgf_denoise_host")

    def render_host(self, gbuffer, image: np.ndarray) -> None:
        """Host arrays in, the denoised image written back into `image`; blocking."""
        for a in gbuffer:
            assert a.dtype == np.float32 and a.flags.c_contiguous and a.shape == (self.height, self.width, 4)
        assert image.dtype == np.uint8 and image.flags.c_contiguous and image.shape == (self.height, self.width, 4)
        self.render_host_ptr(*(a.ctypes.data for a in gbuffer), image.ctypes.data)

    def profile_frame(self, gbuffer, image, stream=None):
        """One eager frame on device tensors; returns (ms temporal, ms a-trous + copy)."""
        ms = (ctypes.c_double * 2)()
        st = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        self._check(self._lib.neon_svgf_profile_frame(self._h, *(ctypes.c_void_p(t.data_ptr()) for t in gbuffer),
                                                      ctypes.c_void_p(image.data_ptr()), ms, st), "neon_svgf_profile_frame")
        return float(ms[0]), float(ms[1])

    def read_state(self):
        """(colour_a, colour_b, moments, ping_pong) as host arrays."""
        h, w = self.height, self.width
        a, b, m = np.empty((h, w, 4), np.uint16), np.empty((h, w, 4), np.uint16), np.empty((h, w, 4), np.float32)
        for name, arr in (("colour_a", a), ("colour_b", b), ("moments", m)):
            self._check(self._lib.neon_svgf_read(self._h, name.encode(), ctypes.c_void_p(arr.ctypes.data), arr.nbytes), "neon_svgf_read")
        pp = ctypes.c_int32()
        self._check(self._lib.neon_svgf_read(self._h, b"ping_pong", ctypes.byref(pp), 4), "neon_svgf_read")
        return a, b, m, int(pp.value)

    def set_option(self, name: str, value: int) -> None:
        self._check(self._lib.neon_svgf_set_option(self._h, name.encode(), int(value)), "neon_svgf_set_option")

    def launch_count(self) -> int:
        return int(self._lib.neon_svgf_launch_count(self._h))

    def close(self) -> None:
        if self._h:
            self._lib.neon_svgf_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
