"""Path-tracer oracles on the CPU: the plain-C restatement (oracle/pt_oracle.c) must reproduce, bit for
bit, the committed frames that the reference engine's own shaders produced when compiled for the CPU
(tests/golden/pt_small.npz, made by tests/golden/make_pt_golden.py), and those shaders themselves where
the compiled library is present.  Also: the scene generator's invariants and the C ABI's argument checks
(no GPU needed)."""
import ctypes
import os

import numpy as np
import pytest

from neonengine_b200 import _lib, pt_synth
from oracle import pt

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pt_small.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.mark.parametrize("name", ["small_seed1", "small_seed4"])
def test_restatement_reproduces_the_reference_shaders_fixture(golden, name):
    seed, w, h, frame_id = golden[name + "_params"]
    sc = pt_synth.small_scene(int(seed))
    ip, iv = pt_synth.camera(int(w), int(h))
    img, rays = pt.render(sc, ip, iv, float(frame_id), int(w), int(h))
    np.testing.assert_array_equal(img, golden[name + "_image"])
    assert rays == int(golden[name + "_rays"])
    # every material type is on some path of these frames, and the frame is not flat
    assert len(np.unique(img.reshape(-1, 4), axis=0)) > 100


def test_restatement_equals_compiled_reference_shaders_where_present():
    if not pt.have_ref():
        pytest.skip("the compiled reference shaders are not available here")
    for sc, (w, h), fid in ((pt_synth.small_scene(9), (64, 40), 0.0), (pt_synth.cornell_box(3), (160, 120), 21.0)):
        ip, iv = pt_synth.camera(w, h, rotation=(0.1, -0.2, 0.05))
        a, ra = pt.ref_render(sc, ip, iv, fid, w, h)
        b, rb = pt.render(sc, ip, iv, fid, w, h)
        np.testing.assert_array_equal(a, b)
        assert ra == rb


def test_cornell_crop_of_the_engine_configuration(golden):
    """Rows 300..307 of the 800 x 600 Cornell frame: rendering only needs those rows' pixels, but every
    pixel is independent, so the restatement renders the whole frame at a reduced cost by ... rendering it."""
    sc = pt_synth.cornell_box(0)
    ip, iv = pt_synth.camera(800, 600)
    img, rays = pt.render(sc, ip, iv, 5.0, 800, 600)
    np.testing.assert_array_equal(img[300:308], golden["cornell_rows_300_308"])
    assert rays == int(golden["cornell_rays"]) and int(img.astype(np.int64).sum()) == int(golden["cornell_checksum"])


def test_scene_generator_invariants():
    sc = pt_synth.cornell_box(0)
    assert sc.n_lights == 50 and len(sc.materials) == 54
    assert (sc.vertices["material"][: 10] == 0).all() and sc.indices.max() < len(sc.vertices)
    assert np.allclose(np.linalg.norm(sc.vertices["normal"][:, :3], axis=1), 1.0, atol=1e-6)
    # lights carry emission and their centre + sampling radius; walls do not emit
    assert (sc.materials["emission"][:50, 0] == 30).all() and (sc.materials["emission"][50:] == 0).all()
    assert (sc.materials["position"][:50, 3] == np.float32(0.1)).all()
    # outward winding: the geometric normal of every cube triangle agrees with its vertex normals
    v, i = sc.vertices, sc.indices.reshape(-1, 3)
    cube = v["material"][i[:, 0]] >= 50
    p0, p1, p2 = (v["pos"][i[cube, k], :3] for k in range(3))
    gn = np.cross(p1 - p0, p2 - p0)
    assert (np.einsum("ij,ij->i", gn, v["normal"][i[cube, 0], :3]) > 0).all()
    ip, iv = pt_synth.camera(800, 600)
    assert ip.shape == (16,) and iv[12:15].tolist() == pytest.approx([0.0444, -0.7041, -1.1978])


def test_pt_create_rejects_bad_arguments():
    lib = _lib.load()
    sc = pt_synth.small_scene(1)
    h = ctypes.c_void_p()
    cfg = _lib.NeonPtConfig(0, 10, 6, 0)
    v, i, m = sc.vertices, sc.indices, sc.materials
    assert lib.neon_pt_create(ctypes.byref(cfg), v.ctypes.data, len(v), i.ctypes.data, len(i), m.ctypes.data, len(m), ctypes.byref(h)) == 1
    assert b"image size" in lib.neon_pt_last_error(None)
    cfg = _lib.NeonPtConfig(16, 16, 6, 0)
    bad = i.copy()
    bad[5] = len(v) + 3
    assert lib.neon_pt_create(ctypes.byref(cfg), v.ctypes.data, len(v), bad.ctypes.data, len(bad), m.ctypes.data, len(m), ctypes.byref(h)) == 1
    assert b"refers to vertex" in lib.neon_pt_last_error(None)
    cfg = _lib.NeonPtConfig(16, 16, 99, 0)
    assert lib.neon_pt_create(ctypes.byref(cfg), v.ctypes.data, len(v), i.ctypes.data, len(i), m.ctypes.data, len(m), ctypes.byref(h)) == 1
    assert lib.neon_pt_render(None, None, None, ctypes.c_float(0), None, None) == 1
