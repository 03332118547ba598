"""Procedural scene and camera for the path tracer: the reference engine's Cornell box.

`RayTracingApp::buildCornellBox` (NeonEngine/src/raytracing_app.cpp:928-1025) places 50 sphere lights
(sphere.obj scaled to radius 0.075, emission 30, light radius 0.1 for the sampler) on a jittered ring at
y = -3 and four scaled copies of cube.obj (floor, right wall, left wall, back wall); the app flattens every
object's mesh into one world-space vertex / index list with materialIndex = object id
(raytracing_app.cpp:151-176) and builds the material buffer with the lights first
(raytracing_system.cpp:619-645).  The checkout ships neither .obj file (they are git-ignored), so a
generated [-1, 1]^3 cube (24 vertices, flat normals) and a unit UV sphere (smooth normals) stand in; the
engine's rand() becomes a seeded generator.  Triangles are wound counter-clockwise seen from outside.

The camera is LveCamera (NeonEngine/src/lve_camera.cpp:27-47 perspective, :87-124 YXZ view) at the app's
start position (raytracing_app.cpp:596-597), 50 degrees, aspect width / height.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np

VERTEX_DTYPE = np.dtype([("pos", np.float32, 4), ("normal", np.float32, 4), ("uv", np.float32, 4),
                         ("material", np.uint32), ("pad", np.uint32, 3)])
MATERIAL_DTYPE = np.dtype([("emission", np.float32, 4), ("albedo", np.float32, 4), ("position", np.float32, 4),
                           ("misc", np.float32, 4)])


def cube_mesh():
    """[-1, 1]^3, 6 faces x 4 vertices, flat normals, counter-clockwise from outside."""
    pos, nrm, uv, idx = [], [], [], []
    for axis in range(3):
        for sign in (-1.0, 1.0):
            n = [0.0, 0.0, 0.0]
            n[axis] = sign
            a, b = (axis + 1) % 3, (axis + 2) % 3
            base = len(pos)
            for (ca, cb) in ((-1, -1), (1, -1), (1, 1), (-1, 1)):
                p = [0.0, 0.0, 0.0]
                p[axis] = sign
                p[a], p[b] = ca, cb
                pos.append(p)
                nrm.append(n)
                uv.append([(ca + 1) / 2, (cb + 1) / 2])
            quad = [0, 1, 2, 0, 2, 3] if sign > 0 else [0, 2, 1, 0, 3, 2]
            idx += [base + q for q in quad]
    return np.array(pos, np.float32), np.array(nrm, np.float32), np.array(uv, np.float32), np.array(idx, np.uint32)


def sphere_mesh(segments=16, rings=8):
    """Unit UV sphere, smooth normals, counter-clockwise from outside."""
    pos, uv = [], []
    for r in range(rings + 1):
        th = math.pi * r / rings
        for s in range(segments + 1):
            ph = 2 * math.pi * s / segments
            pos.append([math.sin(th) * math.cos(ph), math.cos(th), math.sin(th) * math.sin(ph)])
            uv.append([s / segments, r / rings])
    idx = []
    for r in range(rings):
        for s in range(segments):
            a = r * (segments + 1) + s
            b = a + segments + 1
            if r != 0:
                idx += [a, a + 1, b]
            if r != rings - 1:
                idx += [a + 1, b + 1, b]
    pos = np.array(pos, np.float32)
    return pos, pos.copy(), np.array(uv, np.float32), np.array(idx, np.uint32)


@dataclasses.dataclass
class PtScene:
    vertices: np.ndarray     # VERTEX_DTYPE
    indices: np.ndarray      # uint32, 3 per triangle
    materials: np.ndarray    # MATERIAL_DTYPE, lights first
    n_lights: int


def _place(mesh, translation, scale, obj_id):
    pos, nrm, uv, idx = mesh
    scale = np.asarray(scale, np.float32)
    v = np.zeros(len(pos), VERTEX_DTYPE)
    v["pos"][:, :3] = pos * scale + np.asarray(translation, np.float32)
    v["pos"][:, 3] = 1.0
    n = nrm / scale                                  # transpose(inverse(M)) of a scale-only matrix
    v["normal"][:, :3] = (n / np.linalg.norm(n, axis=1, keepdims=True)).astype(np.float32)
    v["normal"][:, 3] = 1.0
    v["uv"][:, :2] = uv
    v["material"] = obj_id
    return v, idx


def cornell_box(seed: int = 0, n_lights: int = 50, sphere_segments: int = 16, sphere_rings: int = 8) -> PtScene:
    rng = np.random.Generator(np.random.PCG64(seed))
    cube, sphere = cube_mesh(), sphere_mesh(sphere_segments, sphere_rings)
    verts, inds, mats, offset = [], [], [], 0
    ring, y, light_radius = 4.0, -3.0, 0.1

    def add(mesh, translation, scale, mat):
        nonlocal offset
        v, i = _place(mesh, translation, scale, len(mats))
        verts.append(v)
        inds.append(i + offset)
        offset += len(v)
        mats.append(mat)

    for i in range(n_lights):
        ang = np.float32(2.0 * 3.1415927 * i / n_lights)
        x = np.float32(math.cos(ang)) * np.float32(ring) * np.float32(rng.random() * 2.0)
        z = np.float32(math.sin(ang)) * np.float32(ring) * np.float32(rng.random() * 2.0)
        m = np.zeros((), MATERIAL_DTYPE)
        m["emission"] = (30.0, 30.0, 30.0, light_radius * light_radius * 3.1415927 * 4)
        m["albedo"] = 1.0
        m["position"] = (x, y, z, light_radius)
        m["misc"] = (0.5, 0.0, 0.0, 0.0)
        add(sphere, (x, y, z), (light_radius * 0.75,) * 3, m)

    def wall():
        m = np.zeros((), MATERIAL_DTYPE)
        m["albedo"] = 1.0
        m["misc"] = (1.0, 0.0, 0.0, 0.0)
        return m

    add(cube, (0.0, -0.5, 0.0), (0.58, 0.04, 0.5), wall())      # floor
    add(cube, (0.54, -1.0, 0.0), (0.04, 0.46, 0.5), wall())     # right wall
    add(cube, (-0.54, -1.0, 0.0), (0.04, 0.46, 0.5), wall())    # left wall
    add(cube, (0.0, -1.0, 0.5), (0.5, 0.5, 0.04), wall())       # back wall
    return PtScene(np.concatenate(verts), np.concatenate(inds).astype(np.uint32), np.array(mats, MATERIAL_DTYPE), n_lights)


def small_scene(seed: int = 1) -> PtScene:
    """A quick test scene: the box with 6 lights close above it, one mirror-like wall and a glass block."""
    rng = np.random.Generator(np.random.PCG64(seed))
    sc = cornell_box(seed, n_lights=6, sphere_segments=8, sphere_rings=4)
    mats = sc.materials.copy()
    for i in range(6):
        mats[i]["position"][:3] = (rng.uniform(-0.4, 0.4), -1.9, rng.uniform(-0.3, 0.3))
    verts = sc.vertices.copy()
    # move the light meshes to their new centres
    for i in range(6):
        sel = verts["material"] == i
        verts["pos"][sel, :3] += mats[i]["position"][:3] - sc.materials[i]["position"][:3]
    mats[7]["misc"][0] = 0.15            # right wall: mostly mirror
    mats[8]["albedo"][:3] = (0.2, 0.8, 0.3)
    cube = cube_mesh()
    v, i = _place(cube, (0.1, -0.7, 0.1), (0.12, 0.12, 0.12), len(mats))
    glass = np.zeros((), MATERIAL_DTYPE)
    glass["albedo"] = 1.0
    glass["misc"] = (0.0, 1.5, 67.0, 0.0)
    v2, i2 = _place(cube, (-0.25, -0.62, -0.05), (0.08, 0.08, 0.08), len(mats) + 1)
    tex = np.zeros((), MATERIAL_DTYPE)
    tex["albedo"] = 1.0
    tex["misc"] = (0.8, 0.0, 2.0, 0.0)
    n0 = len(verts)
    return PtScene(np.concatenate([verts, v, v2]), np.concatenate([sc.indices, i + n0, i2 + n0 + len(v)]).astype(np.uint32),
                   np.concatenate([mats, np.array([glass, tex], MATERIAL_DTYPE)]), 6)


def camera(width: int, height: int, position=(0.0444, -0.7041, -1.1978), rotation=(0.0, 0.0, 0.0), fovy_deg: float = 50.0):
    """(inverse_projection, inverse_view) as column-major float32[16], as RayUbo holds them."""
    f32 = np.float32
    tan_half = f32(math.tan(f32(math.radians(fovy_deg)) * f32(0.5)))
    aspect = f32(width) / f32(height)
    near, far = f32(0.1), f32(100.0)
    A, B = f32(1.0) / (aspect * tan_half), f32(1.0) / tan_half
    C, D = far / (far - near), -(far * near) / (far - near)
    ip = np.zeros((4, 4), np.float32)        # ip[col][row]
    ip[0][0] = f32(1.0) / A
    ip[1][1] = f32(1.0) / B
    ip[2][3] = f32(1.0) / D
    ip[3][2] = 1.0
    ip[3][3] = -C / D
    c3, s3 = f32(math.cos(rotation[2])), f32(math.sin(rotation[2]))
    c2, s2 = f32(math.cos(rotation[0])), f32(math.sin(rotation[0]))
    c1, s1 = f32(math.cos(rotation[1])), f32(math.sin(rotation[1]))
    u = (c1 * c3 + s1 * s2 * s3, c2 * s3, c1 * s2 * s3 - c3 * s1)
    v = (c3 * s1 * s2 - c1 * s3, c2 * c3, c1 * c3 * s2 + s1 * s3)
    w = (c2 * s1, -s2, c1 * c2)
    iv = np.eye(4, dtype=np.float32)
    iv[0][:3], iv[1][:3], iv[2][:3] = u, v, w
    iv[3][:3] = position
    return ip.reshape(16).copy(), iv.reshape(16).copy()
