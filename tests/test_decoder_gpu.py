"""GPU parity of the decoder stack (include/neon_decoder.h) against oracle/decoder_oracle.py.

Tolerances (stated here because the MoE contract covers the MoE output only): fp32
intermediates (q, residual stream, logits) within 2e-2 absolute and 5e-3 mean relative like
the MoE contract; bf16 tensors within one bf16 step (2^-7 relative) of the oracle's value.
Routing is compared on equal inputs: the oracle's MoE receives the device's own bf16 input.
"""
import dataclasses

import numpy as np
import pytest

from helpers import MAX_ABS_TOL, MEAN_REL_TOL, errors

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _setup(shape, B, ctx, seed, share_moe=False):
    import oracle
    from neonengine_b200.decoder_synth import make_decoder_weights, make_kv
    from neonengine_b200.decoder_system import DecoderSystem
    w = make_decoder_weights(shape, seed, share_moe=share_moe)
    sys_ = DecoderSystem(shape, B, ctx)
    sys_.set_weights(w)
    kc, vc = [], []
    for l in range(shape.n_layers):
        k, v = make_kv(shape, l, B, ctx, seed)
        sys_.load_kv(l, k, v)
        kc.append(k.copy())
        vc.append(v.copy())

    def moe_fn(l, xn_bits):
        return oracle.moe_forward(np.ascontiguousarray(xn_bits), w.moe[l])[0]
    return w, sys_, kc, vc, moe_fn


def _bf16_close(got_bits, ref_bits, what, floor=1e-2):
    """Within one bf16 step of the oracle's value; `floor` is the magnitude below which the
    step of `floor` itself is allowed (fp32 noise on near-zero elements of a normalised row)."""
    from neonengine_b200.synth import bf16_bits_to_f32
    g, r = bf16_bits_to_f32(got_bits).astype(np.float64), bf16_bits_to_f32(ref_bits).astype(np.float64)
    tol = np.maximum(np.abs(r), floor) * 2.0 ** -7 * 1.01
    bad = np.abs(g - r) > tol
    assert not bad.any(), f"{what}: {bad.sum()} elements beyond one bf16 step, worst {np.abs(g - r).max()}"


def _small_shape(n_layers=2, window=8):
    from neonengine_b200.decoder_synth import DecoderShape
    from neonengine_b200.synth import MoeShape
    return DecoderShape(n_layers=n_layers, hidden=256, n_q_heads=8, n_kv_heads=2, vocab=512, window=window,
                        moe=MoeShape(hidden=256, inter=128, n_experts=8, top_k=4))


def test_yarn_frequencies_match_oracle():
    from oracle import decoder_oracle as dor
    from neonengine_b200.decoder_system import DecoderSystem
    for factor in (1.0, 32.0):
        shape = dataclasses.replace(_small_shape(1), rope_factor=factor)
        s = DecoderSystem(shape, 1, 16)
        inv, _ = dor.yarn_inv_freq(shape)
        np.testing.assert_array_equal(s.read("inv_freq"), inv)
        s.close()


@pytest.mark.parametrize("B,positions", [(3, [5, 31, 17]), (1, [0]), (8, [31, 30, 29, 7, 8, 9, 0, 15])])
def test_small_decoder_step_matches_oracle(B, positions):
    from oracle import decoder_oracle as dor
    shape = _small_shape()
    ctx = 32
    w, s, kc, vc, moe_fn = _setup(shape, B, ctx, seed=11)
    tokens = np.arange(7, 7 + B, dtype=np.int32) * 13 % shape.vocab
    pos = np.asarray(positions, np.int32)
    t_dev, p_dev = torch.from_numpy(tokens).cuda(), torch.from_numpy(pos).cuda()
    nxt = torch.zeros(B, dtype=torch.int32, device="cuda")
    # layer by layer: feed the oracle the device's own MoE input so routing sees equal bits
    override = {}
    for l in range(shape.n_layers):
        s.set_option("stop_after_layer", l + 1)
        s.step(t_dev, p_dev)
        override[l] = s.read("moe_in", B)
    s.set_option("stop_after_layer", 0)
    s.step(t_dev, p_dev, next_tokens=nxt)
    ref = dor.decoder_step(w, kc, vc, tokens, pos, moe_fn, moe_in_override=override)
    qkv = s.read("qkv", B)
    nq, D = shape.n_q_heads, shape.head_dim
    ea, er = errors(qkv[:, :nq * D], ref["q"].reshape(B, -1))
    assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
    from neonengine_b200.synth import bf16_bits_to_f32 as f
    # downstream of layer 0's MoE the inputs already differ within the MoE tolerance
    ea, er = errors(f(s.read("attn", B)), f(ref["attn"]))
    assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
    ea, er = errors(f(s.read("moe_in", B)), f(dor.rmsnorm(ref["x_mid"], w.attention[-1].ln2, shape.rms_eps)))
    assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
    ea, er = errors(s.read("moe_out", B), ref["moe_out"])
    assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
    ea, er = errors(s.read("x", B), ref["x"])
    assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
    logits = s.read("logits", B)
    ea, er = errors(logits, ref["logits"])
    assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
    # argmax: equal wherever the oracle's best logit leads by more than the tolerance
    top2 = np.sort(ref["logits"], axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 2 * MAX_ABS_TOL
    np.testing.assert_array_equal(nxt.cpu().numpy()[clear], ref["next"][clear])
    np.testing.assert_array_equal(nxt.cpu().numpy(), np.argmax(logits, axis=-1))
    s.close()


def test_cache_append_and_window():
    """The step writes the new K/V at its position; an even (windowed) layer ignores older
    positions, an odd layer does not."""
    shape = _small_shape(n_layers=2, window=4)
    B, ctx = 2, 32
    w, s, kc, vc, moe_fn = _setup(shape, B, ctx, seed=5)
    tokens = torch.tensor([3, 4], dtype=torch.int32, device="cuda")
    pos = torch.tensor([20, 9], dtype=torch.int32, device="cuda")
    s.set_option("stop_after_layer", 1)
    s.step(tokens, pos)
    a0 = s.read("attn", B).copy()
    # scramble cache rows outside the window of layer 0 (positions < p - 3): no effect
    from neonengine_b200.decoder_synth import make_kv
    k2, v2 = make_kv(shape, 0, B, 5, base_seed=99)
    s.load_kv(0, k2, v2)  # overwrites positions 0..4 of both sequences
    s.step(tokens, pos)
    np.testing.assert_array_equal(s.read("attn", B), a0)
    s.close()
    # without a window the same overwrite changes the result
    shape_nw = dataclasses.replace(shape, window=0)
    w, s, kc, vc, moe_fn = _setup(shape_nw, B, ctx, seed=5)
    s.set_option("stop_after_layer", 1)
    s.step(tokens, pos)
    a0 = s.read("attn", B).copy()
    s.load_kv(0, k2, v2)
    s.step(tokens, pos)
    assert (s.read("attn", B) != a0).any()
    s.close()


def test_graph_replay_and_host_step_agree():
    shape = _small_shape()
    B, ctx = 4, 32
    w, s, kc, vc, moe_fn = _setup(shape, B, ctx, seed=3)
    tokens = np.array([1, 2, 3, 4], np.int32)
    pos = np.array([31, 12, 0, 7], np.int32)
    t_dev, p_dev = torch.from_numpy(tokens).cuda(), torch.from_numpy(pos).cuda()
    outs = []
    for _ in range(4):  # eager, capture, replay, replay
        nxt = torch.zeros(B, dtype=torch.int32, device="cuda") if not outs else nxt
        s.step(t_dev, p_dev, next_tokens=nxt)
        torch.cuda.synchronize()
        outs.append((nxt.cpu().numpy().copy(), s.read("logits", B).copy()))
    for n, lg in outs[1:]:
        np.testing.assert_array_equal(n, outs[0][0])
        np.testing.assert_array_equal(lg, outs[0][1])
    np.testing.assert_array_equal(s.step_host(tokens, pos), outs[0][0])
    before = s.launch_count()
    s.step_host(tokens, pos)
    assert s.launch_count() > before
    s.close()


def test_rejects_bad_arguments():
    shape = _small_shape(1)
    from neonengine_b200.decoder_system import DecoderSystem
    s = DecoderSystem(shape, 2, 16)
    t = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="set_embeddings"):
        s.step(t, t)
    with pytest.raises(RuntimeError):
        s.set_option("nonsense", 1)
    s.close()


def test_full_width_layer_matches_oracle():
    """One layer at the real widths (hidden 2880, 64/8 heads, 32 experts, 4096-token cache,
    batch 8), small vocabulary; layer 0 is windowed, so a second run with window 0 covers
    full attention over the whole cache."""
    from oracle import decoder_oracle as dor
    from neonengine_b200.decoder_synth import DecoderShape
    for window in (128, 0):
        shape = DecoderShape(n_layers=1, vocab=1024, window=window)
        B, ctx = 8, 4096
        w, s, kc, vc, moe_fn = _setup(shape, B, ctx, seed=21)
        tokens = np.arange(B, dtype=np.int32) * 101 % shape.vocab
        pos = np.array([4095, 4095, 4000, 130, 127, 1, 2047, 4094], np.int32)
        t_dev, p_dev = torch.from_numpy(tokens).cuda(), torch.from_numpy(pos).cuda()
        s.step(t_dev, p_dev)
        override = {0: s.read("moe_in", B)}
        ref = dor.decoder_step(w, kc, vc, tokens, pos, moe_fn, moe_in_override=override)
        nq, D = shape.n_q_heads, shape.head_dim
        ea, er = errors(s.read("qkv", B)[:, :nq * D], ref["q"].reshape(B, -1))
        assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
        _bf16_close(s.read("attn", B), ref["attn"], f"attention output (window {window})")
        _bf16_close(s.read("moe_in", B), dor.rmsnorm(ref["x_mid"], w.attention[0].ln2, shape.rms_eps), "MoE input",
                    floor=0.25)
        ea, er = errors(s.read("moe_out", B), ref["moe_out"])
        assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
        ea, er = errors(s.read("logits", B), ref["logits"])
        assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (ea, er)
        s.close()


def test_generation_over_several_steps_matches_oracle():
    """Three consecutive decode steps with advancing positions: the K/V the earlier steps appended
    are what the later steps attend to.  The oracle follows the device's token choices and, per
    layer, the device's own bf16 MoE input (so routing is compared on equal bits)."""
    from oracle import decoder_oracle as dor
    shape = _small_shape()
    B, ctx = 3, 32
    w, s, kc, vc, moe_fn = _setup(shape, B, ctx, seed=17)
    tokens = np.array([5, 99, 300], np.int32)
    pos = np.array([10, 0, 28], np.int32)
    for step in range(3):
        t_dev, p_dev = torch.from_numpy(tokens).cuda(), torch.from_numpy(pos).cuda()
        nxt = torch.zeros(B, dtype=torch.int32, device="cuda")
        override = {}
        for l in range(shape.n_layers):
            s.set_option("stop_after_layer", l + 1)
            s.step(t_dev, p_dev)
            override[l] = s.read("moe_in", B)
        s.set_option("stop_after_layer", 0)
        s.step(t_dev, p_dev, next_tokens=nxt)
        ref = dor.decoder_step(w, kc, vc, tokens, pos, moe_fn, moe_in_override=override)
        logits = s.read("logits", B)
        ea, er = errors(logits, ref["logits"])
        assert ea <= MAX_ABS_TOL and er <= MEAN_REL_TOL, (step, ea, er)
        got = nxt.cpu().numpy()
        np.testing.assert_array_equal(got, np.argmax(logits, axis=-1))
        tokens, pos = got.astype(np.int32), pos + 1
    s.close()


def test_out_of_range_tokens_and_positions_are_clamped():
    shape = _small_shape(1)
    B, ctx = 2, 16
    w, s, kc, vc, moe_fn = _setup(shape, B, ctx, seed=2)
    good = (torch.tensor([shape.vocab - 1, 0], dtype=torch.int32, device="cuda"),
            torch.tensor([ctx - 1, 0], dtype=torch.int32, device="cuda"))
    bad = (torch.tensor([shape.vocab + 1000, -7], dtype=torch.int32, device="cuda"),
           torch.tensor([ctx + 50, -3], dtype=torch.int32, device="cuda"))
    s.set_option("use_graphs", 0)
    s.step(*good)
    a = s.read("logits", B).copy()
    s.step(*bad)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(s.read("logits", B), a)
    s.close()
