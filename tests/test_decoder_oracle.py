"""CPU tests of the decoder restatement (oracle/decoder_oracle.py): properties the published
algorithms guarantee, checked without a GPU."""
import dataclasses
import math

import numpy as np

from neonengine_b200.decoder_synth import DecoderShape, make_decoder_weights, make_kv
from neonengine_b200.synth import MoeShape, bf16_bits_to_f32, f32_to_bf16_bits
from oracle import decoder_oracle as dor

SHAPE = DecoderShape(n_layers=2, hidden=128, n_q_heads=4, n_kv_heads=2, vocab=64, window=4,
                     moe=MoeShape(hidden=128, inter=64, n_experts=4, top_k=2))


def test_yarn_blends_between_interpolation_and_extrapolation():
    inv, mscale = dor.yarn_inv_freq(DecoderShape())
    plain, one = dor.yarn_inv_freq(dataclasses.replace(DecoderShape(), rope_factor=1.0))
    assert one == 1.0 and abs(mscale - (0.1 * math.log(32.0) + 1.0)) < 1e-6
    np.testing.assert_allclose(plain, 150000.0 ** (-np.arange(32) / 32.0), rtol=1e-6)
    ratio = inv / plain
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 32) < 1e-6       # fastest kept, slowest interpolated
    assert (np.diff(ratio) <= 1e-7).all()                            # monotone ramp in between
    assert ((ratio > 1 / 32 + 1e-4) & (ratio < 1 - 1e-4)).any()


def test_rope_is_a_scaled_rotation_and_relative():
    g = np.random.default_rng(0)
    inv, mscale = dor.yarn_inv_freq(SHAPE)
    q, k = g.normal(size=(1, 1, 64)), g.normal(size=(1, 1, 64))
    for p in (0, 5, 1000):
        r = dor.rope(q, [p], inv, mscale)
        np.testing.assert_allclose(np.linalg.norm(r), mscale * np.linalg.norm(q), rtol=1e-6)
    np.testing.assert_allclose(dor.rope(q, [0], inv, 1.0), q)
    d1 = (dor.rope(q, [17], inv, 1.0) * dor.rope(k, [11], inv, 1.0)).sum()
    d2 = (dor.rope(q, [106], inv, 1.0) * dor.rope(k, [100], inv, 1.0)).sum()
    np.testing.assert_allclose(d1, d2, rtol=1e-4)


def test_rmsnorm_scale_invariance():
    g = np.random.default_rng(1)
    x = g.normal(size=(3, 128))
    w = f32_to_bf16_bits(np.ones(128, np.float32))
    a = bf16_bits_to_f32(dor.rmsnorm(x, w, 0.0))
    b = bf16_bits_to_f32(dor.rmsnorm(x * 64.0, w, 0.0))
    np.testing.assert_array_equal(a, b)
    np.testing.assert_allclose((a.astype(np.float64) ** 2).mean(-1), 1.0, rtol=1e-2)


def test_attention_sink_and_window():
    g = np.random.default_rng(2)
    B, ctx, nq, nkv, D = 2, 16, 4, 2, 64
    q = g.normal(size=(B, nq, D))
    k = f32_to_bf16_bits(g.normal(size=(B, ctx, nkv, D)).astype(np.float32))
    v = f32_to_bf16_bits(g.normal(size=(B, ctx, nkv, D)).astype(np.float32))
    pos = [15, 6]
    minus_inf = f32_to_bf16_bits(np.full(nq, -1e30, np.float32))
    out = dor.attention(q, k, v, pos, minus_inf, 0).reshape(B, nq, D)
    # a sink at -inf leaves an ordinary softmax over positions 0..p
    kf, vf = bf16_bits_to_f32(k).astype(np.float64), bf16_bits_to_f32(v).astype(np.float64)
    s = kf[1, :7, 0] @ q[1, 1] / 8.0
    pr = np.exp(s - s.max()); pr /= pr.sum()
    np.testing.assert_allclose(out[1, 1], pr @ vf[1, :7, 0], rtol=1e-9)
    # a finite sink only shrinks the output: same direction, factor sum/(sum + exp(sink))
    zero = f32_to_bf16_bits(np.zeros(nq, np.float32))
    out0 = dor.attention(q, k, v, pos, zero, 0).reshape(B, nq, D)
    fac = np.exp(s).sum() / (np.exp(s).sum() + 1.0)
    np.testing.assert_allclose(out0[1, 1], out[1, 1] * fac, rtol=1e-9)
    # a window of 3 sees only the last three positions
    outw = dor.attention(q, k, v, pos, minus_inf, 3).reshape(B, nq, D)
    s3 = s[4:7]; p3 = np.exp(s3 - s3.max()); p3 /= p3.sum()
    np.testing.assert_allclose(outw[1, 1], p3 @ vf[1, 4:7, 0], rtol=1e-9)


def test_decoder_step_updates_cache_and_is_deterministic():
    import oracle
    w = make_decoder_weights(SHAPE, 4)
    caches = [make_kv(SHAPE, l, 2, 8, 4) for l in range(2)]
    tokens, pos = np.array([3, 9], np.int32), np.array([7, 2], np.int32)

    def moe_fn(l, xn):
        return oracle.moe_forward(np.ascontiguousarray(xn), w.moe[l])[0]
    outs = []
    for _ in range(2):
        kc, vc = [c[0].copy() for c in caches], [c[1].copy() for c in caches]
        outs.append(dor.decoder_step(w, kc, vc, tokens, pos, moe_fn))
        assert (kc[0][0, 7] != caches[0][0][0, 7]).any() and (kc[0][0, 6] == caches[0][0][0, 6]).all()
        assert (vc[1][1, 2] != caches[1][1][1, 2]).any() and (vc[1][1, 3] == caches[1][1][1, 3]).all()
    np.testing.assert_array_equal(outs[0]["logits"], outs[1]["logits"])
    assert outs[0]["logits"].shape == (2, 64) and np.isfinite(outs[0]["logits"]).all()
