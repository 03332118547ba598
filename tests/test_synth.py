import numpy as np

from neonengine_b200 import synth


def test_bf16_round_trip_and_rounding():
    x = np.array([1.0, -2.5, 3.1415927, 1e-3, 65504.0, 0.0], np.float32)
    b = synth.f32_to_bf16_bits(x)
    back = synth.bf16_bits_to_f32(b)
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)
    # ties to even: 1 + 2^-8 is halfway between 1 and 1 + 2^-7
    assert synth.f32_to_bf16_bits(np.array([1.0 + 2.0 ** -8], np.float32))[0] == 0x3F80


def test_weights_are_seeded_and_shardable():
    sh = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    a = synth.make_weights(sh, 0)
    b = synth.make_weights(sh, 0)
    c = synth.make_weights(sh, 0, experts=(4, 8))
    for name in ("router_w", "gate_up_blocks", "gate_up_scales", "down_bias"):
        np.testing.assert_array_equal(getattr(a, name), getattr(b, name))
    np.testing.assert_array_equal(a.gate_up_blocks[4:8], c.gate_up_blocks)
    np.testing.assert_array_equal(a.down_scales[4:8], c.down_scales)
    assert a.gate_up_scales.min() >= 117 and a.gate_up_scales.max() <= 123
    assert set(np.unique(a.gate_up_blocks & 15)) == set(range(16))


def test_hidden_gap_rule():
    sh = synth.MoeShape(hidden=128, inter=64, n_experts=32, top_k=4)
    W = synth.make_weights(sh, 1)
    lb = synth.zipf_logit_bias(32)
    h = synth.make_hidden(256, W, 1, logit_bias=lb)
    lg = synth.router_logits_f64(h, W, lb)
    top = -np.sort(-lg, axis=1)[:, :5]
    assert (top[:, :-1] - top[:, 1:]).min() >= 1e-4


def test_shape_byte_counts():
    sh = synth.MoeShape()
    assert sh.expert_bytes == 13_236_480
    assert sh.flops_per_pair == 49_766_400
    assert sh.router_bytes == 184_384


def test_dequant_known_values():
    blocks = np.array([[0x21, 0xF7] + [0] * 14], np.uint8)     # codes 1,2,7,15
    scales = np.array([[126]], np.uint8)                        # 2^-1
    v = synth.dequant_mxfp4(blocks, scales)
    np.testing.assert_array_equal(v[0, :4], np.array([0.25, 0.5, 3.0, -3.0], np.float32))
