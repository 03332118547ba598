"""GPU parity of the path tracer: the CUDA kernel, called through the C ABI, must reproduce the CPU
oracle's frames BIT FOR BIT (integer rgba8 output of a chaotic float computation: every float operation
is pinned by the conventions in include/neon_pt.h), on small scenes that reach every material type, on
the committed fixture made by the reference engine's own shaders, and on the engine's configuration
(Cornell box, 50 sphere lights, 800 x 600, one sample per pixel)."""
import os

import numpy as np
import pytest

from neonengine_b200 import pt_synth
from oracle import pt

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pt_small.npz")


def tracer(scene, w, h):
    import torch
    from neonengine_b200.path_tracer import PathTracer
    assert torch.cuda.is_available()
    return PathTracer(scene, w, h, device=0)


@pytest.mark.parametrize("name", ["small_seed1", "small_seed4"])
def test_fixture_of_the_reference_shaders(name):
    z = np.load(GOLDEN)
    seed, w, h, frame_id = z[name + "_params"]
    sc = pt_synth.small_scene(int(seed))
    t = tracer(sc, int(w), int(h))
    ip, iv = pt_synth.camera(int(w), int(h))
    img = t.render_host(ip, iv, float(frame_id))
    np.testing.assert_array_equal(img, z[name + "_image"])
    assert t.rays() == int(z[name + "_rays"]) and t.status() == 0
    t.close()


def test_small_scenes_against_the_oracle_with_a_turned_camera():
    import torch
    for seed, (w, h), fid, rot in ((2, (120, 72), 1.0, (0.15, -0.3, 0.0)), (7, (67, 45), 40.25, (-0.1, 0.2, 0.3))):
        sc = pt_synth.small_scene(seed)
        t = tracer(sc, w, h)
        ip, iv = pt_synth.camera(w, h, rotation=rot)
        want, rays = pt.render(sc, ip, iv, fid, w, h)
        dev = t.render(ip, iv, fid)                       # device-buffer entry point
        torch.cuda.synchronize()
        np.testing.assert_array_equal(dev.cpu().numpy(), want)
        np.testing.assert_array_equal(t.render_host(ip, iv, fid), want)   # host entry point, and a second run: same bits
        assert t.rays() == 2 * rays and t.status() == 0
        t.close()


def test_engine_configuration_cornell_box_800x600():
    sc = pt_synth.cornell_box(0)
    t = tracer(sc, 800, 600)
    ip, iv = pt_synth.camera(800, 600)
    img = t.render_host(ip, iv, 5.0)
    z = np.load(GOLDEN)
    np.testing.assert_array_equal(img[300:308], z["cornell_rows_300_308"])     # the reference shaders' own rows
    assert int(img.astype(np.int64).sum()) == int(z["cornell_checksum"]) and t.rays() == int(z["cornell_rays"])
    want, _ = pt.render(sc, ip, iv, 5.0, 800, 600)                             # the whole frame against the restatement
    np.testing.assert_array_equal(img, want)
    # another frame id gives another sample of the same scene
    other = t.render_host(ip, iv, 6.0)
    assert not np.array_equal(other, img) and abs(other[..., :3].mean() - img[..., :3].mean()) < 3.0
    nodes, depth = t.bvh_info()
    assert nodes > 1000 and depth < 40 and t.status() == 0
    t.close()
