"""CPU tests: the C oracle against the committed golden vectors (made by an independent
numpy float64 restatement) and against that restatement on fresh inputs."""
import sys

import numpy as np
import pytest

import oracle
from helpers import GOLDEN, load_golden
from neonengine_b200 import synth

sys.path.insert(0, GOLDEN)
import numpy_moe  # noqa: E402

CASES = ["small_seeded", "small_seeded_zipf", "integer_kat", "clamp_negative", "all_ties"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_golden(name):
    shape, W, hidden, lb, z = load_golden(name)
    out, idx, w = oracle.moe_forward(hidden, W, logit_bias=lb)
    np.testing.assert_array_equal(idx, z["idx"])
    np.testing.assert_allclose(w, z["w"], rtol=0, atol=1e-7)
    ref = z["out"]
    np.testing.assert_allclose(out, ref, rtol=2e-6, atol=1e-6 * max(1.0, float(np.abs(ref).max())))


def test_integer_kat_by_hand():
    """gate = lin = 64 -> clamp 7; a = 7*sigmoid(1.702*7)*(7+1); y = 64*a; weights sum to 1."""
    shape, W, hidden, lb, z = load_golden("integer_kat")
    out, idx, w = oracle.moe_forward(hidden, W)
    a = 7.0 / (1.0 + np.exp(-1.702 * 7.0)) * 8.0
    np.testing.assert_allclose(out, np.full_like(out, 64.0 * a), rtol=1e-6)
    np.testing.assert_array_equal(idx, np.tile(np.array([3, 2], np.int32), (2, 1)))  # largest rows win
    np.testing.assert_allclose(w.sum(axis=1), 1.0, atol=1e-6)


def test_all_ties_lower_id_wins():
    shape, W, hidden, lb, z = load_golden("all_ties")
    idx, w = oracle.route(hidden, W.router_w, W.router_b, shape.top_k)
    np.testing.assert_array_equal(idx, np.tile(np.arange(shape.top_k, dtype=np.int32), (hidden.shape[0], 1)))
    np.testing.assert_allclose(w, 1.0 / shape.top_k, atol=1e-7)


def test_partial_ties_and_negative_zero():
    """Duplicate router rows tie exactly; a -0.0 logit ties with +0.0."""
    sh = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    W = synth.make_weights(sh, 3)
    W.router_w[5] = W.router_w[1]
    W.router_w[6] = W.router_w[1]
    W.router_b[5] = W.router_b[6] = W.router_b[1]
    hidden = synth.make_hidden(16, W, 3, min_gap=0)
    idx, w, lg = oracle.route(hidden, W.router_w, W.router_b, 4, want_logits=True)
    ridx, rw, rlg = numpy_moe.route(hidden, W.router_w, W.router_b, 4)
    np.testing.assert_array_equal(idx, ridx)
    assert np.array_equal(lg[:, 1], lg[:, 5]) and np.array_equal(lg[:, 1], lg[:, 6])
    for t in range(16):  # among tied experts the lower id comes first
        sel = [int(e) for e in idx[t] if e in (1, 5, 6)]
        assert sel == sorted(sel) and (not sel or sel[0] == 1)


@pytest.mark.parametrize("T,E,k", [(1, 8, 4), (7, 16, 4), (33, 32, 4), (5, 4, 1)])
def test_oracle_vs_numpy_fresh(T, E, k):
    sh = synth.MoeShape(hidden=128, inter=64, n_experts=E, top_k=k)
    W = synth.make_weights(sh, 11 + T)
    hidden = synth.make_hidden(T, W, 11 + T)
    lb = synth.zipf_logit_bias(E) if T % 2 else None
    out, idx, w = oracle.moe_forward(hidden, W, logit_bias=lb)
    Wd = {n: getattr(W, n) for n in ("router_w", "router_b", "gate_up_blocks", "gate_up_scales", "gate_up_bias",
                                     "down_blocks", "down_scales", "down_bias")}
    ref, ridx, rw, _ = numpy_moe.forward(hidden, Wd, logit_bias=lb, k=k)
    np.testing.assert_array_equal(idx, ridx)
    np.testing.assert_allclose(w, rw, atol=1e-7)
    np.testing.assert_allclose(out, ref, rtol=2e-6, atol=1e-6)


def test_token_subset_matches_full():
    sh = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    W = synth.make_weights(sh, 5)
    hidden = synth.make_hidden(12, W, 5)
    full, idx, w = oracle.moe_forward(hidden, W)
    sub = oracle.experts(hidden, idx, w, W, tokens=np.array([9, 0, 4], np.int32))
    np.testing.assert_array_equal(sub, full[[9, 0, 4]])


def test_expert_parallel_partial_sums():
    """Shards of the experts give partial outputs that add up to the full layer."""
    sh = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    W = synth.make_weights(sh, 6)
    hidden = synth.make_hidden(9, W, 6)
    full, idx, w = oracle.moe_forward(hidden, W)
    parts = sum(oracle.experts(hidden, idx, w, W.slice_experts(lo, lo + 4), e_lo=lo).astype(np.float64)
                for lo in (0, 4))
    np.testing.assert_allclose(parts, full, rtol=1e-6, atol=1e-6)


def test_dispatch_stable_counting_sort():
    rng = np.random.default_rng(0)
    for T, k, E in [(1, 4, 32), (64, 4, 32), (300, 4, 128), (5, 2, 4)]:
        idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
        count, offset, perm, inv = oracle.dispatch(idx, E)
        flat = idx.reshape(-1)
        np.testing.assert_array_equal(count, np.bincount(flat, minlength=E))
        np.testing.assert_array_equal(offset, np.concatenate([[0], np.cumsum(count)]))
        np.testing.assert_array_equal(perm, np.argsort(flat, kind="stable"))
        np.testing.assert_array_equal(inv[perm], np.arange(T * k))


def test_swiglu_limits():
    gu = np.array([100.0, 100.0, -100.0, -100.0, 0.0, 0.0, 7.0, -7.0, 3.0, 2.0])
    a = oracle.swiglu(gu)
    sig = lambda v: 1.0 / (1.0 + np.exp(-1.702 * v))
    exp = [7 * sig(7) * 8, -100 * sig(-100) * (-6), 0.0, 7 * sig(7) * (-6), 3 * sig(3) * 3]
    np.testing.assert_allclose(a, exp, rtol=1e-5, atol=1e-300)  # alpha is passed as fp32


def test_quantised_activation_mode_differs_but_is_close():
    sh = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    W = synth.make_weights(sh, 8)
    hidden = synth.make_hidden(4, W, 8)
    exact, idx, w = oracle.moe_forward(hidden, W)
    quant = oracle.experts(hidden, idx, w, W, quant_act=True)
    rel = np.abs(quant - exact).mean() / np.abs(exact).mean()
    assert 1e-3 < rel < 0.5
