"""CPU tests of the denoiser restatement (oracle/svgf_oracle.c): pinned bit for bit against the
fixture the reference engine's own shaders produced (tests/golden/svgf_small.npz, made by
tests/golden/make_svgf_golden.py) and, where the compiled reference shaders are present
(oracle/_ref/libsvgf_ref.so), against them directly at the reference's window size."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))

import make_svgf_golden as golden  # noqa: E402
from neonengine_b200 import svgf_synth  # noqa: E402
from oracle import svgf  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "svgf_small.npz")


def test_synthetic_frames_are_seeded_and_reprojectable():
    g0, im0 = svgf_synth.make_frame(64, 48, 2)
    g1, im1 = svgf_synth.make_frame(64, 48, 2)
    for a, b in zip(g0, g1):
        np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(im0, im1)
    pos, nrm, bary, mot = g0
    hit = (pos[..., :3] ** 2).sum(-1) >= 1e-6
    assert 0.5 < hit.mean() < 0.95                      # sky present, most pixels covered
    assert set(np.unique(nrm[..., 3])) == {0.0, 1.0, 2.0, 3.0, 4.0}
    assert np.abs(mot[hit][:, 0]).max() > 0             # the camera moved


def test_restatement_reproduces_reference_fixture_bit_for_bit():
    z = np.load(GOLDEN)
    st = svgf.State.zeros(golden.W, golden.H)
    for i in range(golden.FRAMES):
        g, image = svgf_synth.make_frame(golden.W, golden.H, i)
        svgf.frame(g, image, st, golden.ITERATIONS, serial=True)
        np.testing.assert_array_equal(image, z[f"image{i}"])
    np.testing.assert_array_equal(st.colour_a, z["colour_a"])
    np.testing.assert_array_equal(st.colour_b, z["colour_b"])
    np.testing.assert_array_equal(st.data.view(np.uint32), z["moments"].view(np.uint32))
    assert st.ping_pong == int(z["ping_pong"][0])
    assert (st.data[..., 0] > 1).mean() > 0.5           # history was found and accumulated


@pytest.mark.skipif(not svgf.have_ref(), reason="compiled reference shaders not present")
@pytest.mark.parametrize("iterations", [3, 2, 0])
def test_restatement_equals_compiled_reference_shaders(iterations):
    w, h = (800, 600) if iterations == 3 else (200, 120)
    a, b = svgf.State.zeros(w, h), svgf.State.zeros(w, h)
    for i in range(3):
        g, image = svgf_synth.make_frame(w, h, i)
        ia, ib = image.copy(), image.copy()
        svgf.frame(g, ia, a, iterations, serial=True)
        svgf.ref_frame(g, ib, b, iterations)
        np.testing.assert_array_equal(ia, ib)
        np.testing.assert_array_equal(a.colour_a, b.colour_a)
        np.testing.assert_array_equal(a.colour_b, b.colour_b)
        np.testing.assert_array_equal(a.data.view(np.uint32), b.data.view(np.uint32))
        assert a.ping_pong == b.ping_pong


@pytest.mark.skipif(not svgf.have_ref(), reason="compiled reference shaders not present")
def test_shaders_as_shipped_do_nothing():
    """Both shaders start with `return;` in the checkout: a frame only flips the ping-pong flag."""
    g, image = svgf_synth.make_frame(64, 48, 1)
    st, before = svgf.State.zeros(64, 48), image.copy()
    svgf.ref_frame(g, image, st, 3, honour_early_return=True)
    np.testing.assert_array_equal(image, before)
    assert not st.colour_a.any() and not st.colour_b.any() and not st.data.any() and st.ping_pong == 1


def test_snapshot_rule_differs_from_serial_only_through_the_moments_race():
    """Frame 0 has no history and zero variance everywhere the filter looks, so both rules agree;
    later frames differ slightly (the in-place variance a neighbour reads)."""
    w, h = 96, 64
    a, b = svgf.State.zeros(w, h), svgf.State.zeros(w, h)
    g, image = svgf_synth.make_frame(w, h, 0)
    ia, ib = image.copy(), image.copy()
    svgf.frame(g, ia, a, 3, serial=True)
    svgf.frame(g, ib, b, 3, serial=False)
    np.testing.assert_array_equal(a.data[..., :3], b.data[..., :3])   # history length and moments never race
    g, image = svgf_synth.make_frame(w, h, 1)
    ia, ib = image.copy(), image.copy()
    svgf.frame(g, ia, a, 3, serial=True)
    svgf.frame(g, ib, b, 3, serial=False)
    assert np.abs(ia.astype(int) - ib.astype(int)).max() <= 8


def test_denoiser_reduces_noise():
    w, h = 160, 96
    st = svgf.State.zeros(w, h)
    for i in range(4):
        g, image = svgf_synth.make_frame(w, h, i)
        clean = svgf_synth.make_frame(w, h, i, noise=0.0)[1]
        noisy_err = np.abs(image[..., :3].astype(float) - clean[..., :3]).mean()
        svgf.frame(g, image, st, 3)
        err = np.abs(image[..., :3].astype(float) - clean[..., :3]).mean()
    assert err < 0.35 * noisy_err


def test_exp2_polynomial_accuracy():
    xs = np.concatenate([np.linspace(-125.9, 0, 4001), -np.logspace(-8, 1, 500)]).astype(np.float32)
    mine = np.array([svgf.exp2(float(x)) for x in xs])
    exact = np.exp2(xs.astype(np.float64))
    assert (np.abs(mine - exact) / exact).max() < 1.2e-7
    assert svgf.exp2(-200.0) == 0.0 and svgf.exp2(0.0) == 1.0 and svgf.exp2(-1.0) == 0.5
