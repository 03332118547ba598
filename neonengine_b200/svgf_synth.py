"""Seeded synthetic frames for the denoiser: what the engine's G-buffer raster pass and path tracer
hand to the temporal and a-trous passes (NeonEngine/src/raytracing_app.cpp:702-765).

A small analytic scene (floor, a back wall of finite height, two spheres; sky above the wall) is
ray-cast in numpy from a camera that slides sideways a little every frame.  Per frame:
position (camera space, w = 1; all zero where the ray hits nothing), normal (w = mesh id),
barycentric (a smooth stand-in, w = 0), motion (current uv minus the uv the same surface point had
in the previous frame) - four float32 [h, w, 4] images as the engine's rgba32f attachments
(NeonEngine/src/raytracing_rast.cpp:120-123) - and a noisy rgba8 radiance image as the storage
image the path tracer writes (NeonEngine/src/raytracing_system.cpp:517).
"""
from __future__ import annotations

import numpy as np

ALBEDO = np.array([[0, 0, 0], [0.7, 0.7, 0.65], [0.3, 0.5, 0.8], [0.9, 0.3, 0.2], [0.3, 0.8, 0.3]], np.float32)
SKY = np.array([0.35, 0.55, 0.9], np.float32)


def _cast(w: int, h: int, cam_x: float):
    """Nearest hit per pixel: camera-space position, normal, mesh id (0 = nothing)."""
    f = 1.2
    xs = ((np.arange(w, dtype=np.float64) + 0.5) / w - 0.5) * (w / h) / f * 2 * 0.5
    ys = (0.5 - (np.arange(h, dtype=np.float64) + 0.5) / h) / f
    dx, dy = np.meshgrid(xs, ys)
    d = np.stack([dx, dy, -np.ones_like(dx)], -1)
    d /= np.linalg.norm(d, axis=-1, keepdims=True)
    t_best = np.full((h, w), np.inf)
    nrm = np.zeros((h, w, 3))
    mesh = np.zeros((h, w), np.int32)
    o = np.array([cam_x, 0.0, 0.0])

    def take(t, n, ident, ok):
        nonlocal t_best, nrm, mesh
        hit = ok & (t > 1e-3) & (t < t_best)
        t_best = np.where(hit, t, t_best)
        nrm = np.where(hit[..., None], n, nrm)
        mesh = np.where(hit, ident, mesh)

    with np.errstate(divide="ignore", invalid="ignore"):
        t = (-1.0 - o[1]) / d[..., 1]                                   # floor y = -1
        take(t, np.array([0.0, 1.0, 0.0]), 1, np.isfinite(t) & ((o[2] + t * d[..., 2]) > -7.0))
        t = (-7.0 - o[2]) / d[..., 2]                                   # wall z = -7 up to y = 1.2
        take(t, np.array([0.0, 0.0, 1.0]), 2, np.isfinite(t) & ((o[1] + t * d[..., 1]) < 1.2))
        for ident, c, r in ((3, np.array([-0.8, -0.4, -4.0]), 0.6), (4, np.array([1.1, -0.55, -3.2]), 0.45)):
            oc = o - c
            b = (d * oc).sum(-1)
            disc = b * b - ((oc * oc).sum() - r * r)
            t = -b - np.sqrt(np.maximum(disc, 0.0))
            p = o + t[..., None] * d
            take(t, (p - c) / r, ident, disc > 0)
    hit = mesh > 0
    world = np.where(hit[..., None], o + np.where(hit, t_best, 0.0)[..., None] * d, 0.0)
    cam = np.where(hit[..., None], world - o, 0.0)
    return cam, world, nrm, mesh, hit, f


def make_frame(w: int, h: int, index: int, seed: int = 0, pan: float = 0.01, noise: float = 0.15):
    """Returns ((position, normal, barycentric, motion), image) of frame `index`."""
    cam, world, nrm, mesh, hit, f = _cast(w, h, pan * index)
    position = np.zeros((h, w, 4), np.float32)
    position[..., :3] = cam
    position[..., 3] = hit
    normal = np.zeros((h, w, 4), np.float32)
    normal[..., :3] = nrm
    normal[..., 3] = mesh
    bary = np.zeros((h, w, 4), np.float32)
    bary[..., :3] = np.where(hit[..., None], 0.5 + 0.3 * np.sin(0.5 * world + np.array([0.0, 1.0, 2.0])), 0.0)
    # where the same surface point was on screen one frame earlier (camera `pan` further left)
    prev_cam = cam + np.array([pan if index > 0 else 0.0, 0.0, 0.0])
    z = np.where(hit, -prev_cam[..., 2], 1.0)
    prev_u = 0.5 + prev_cam[..., 0] / z * f * (h / w)
    prev_v = 0.5 - prev_cam[..., 1] / z * f
    u = (np.arange(w) + 0.5) / w
    v = (np.arange(h) + 0.5) / h
    motion = np.zeros((h, w, 4), np.float32)
    motion[..., 0] = np.where(hit, u[None, :] - prev_u, 0.0)
    motion[..., 1] = np.where(hit, v[:, None] - prev_v, 0.0)
    light = np.array([0.4, 0.8, 0.45])
    light /= np.linalg.norm(light)
    shade = np.maximum((nrm * light).sum(-1), 0.1)[..., None] * ALBEDO[mesh]
    radiance = np.where(hit[..., None], shade, SKY)
    rng = np.random.Generator(np.random.PCG64(seed * 1000003 + index))
    radiance = radiance + noise * rng.standard_normal((h, w, 3)) * hit[..., None]
    image = np.full((h, w, 4), 255, np.uint8)
    image[..., :3] = np.rint(np.clip(radiance, 0.0, 1.0) * 255.0).astype(np.uint8)
    return (position, normal, bary, motion), image
