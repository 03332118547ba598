"""Generates tests/golden/*.npz.  Run from the repo root: ``python tests/golden/make_golden.py``.

The vectors are produced by numpy_moe.py (float64, independent of the C oracle and of the
CUDA kernels).  The nominal reference engine holds no vectors for this path, so these
pin the oracle only against a second restatement of the same specification.
Cases:
  small_seeded   H=I=64, E=8, k=4, T=6, seeded random inputs in the benchmark distributions
  integer_kat    H=I=64, E=4, k=2, T=2: all weights code 2 (=1.0), scales 2^0, biases 0,
                 hidden = 1.0 -> gate = lin = 64, clamped to 7: a = 7*sigmoid(11.914)*8,
                 y = 64*a; hand-computable.
  all_ties       router weights and bias zero -> every logit 0 -> experts 0..k-1, w = 1/k
  clamp_negative hidden = -1.0 on the integer case -> gate=-64 (unclamped below), lin=-7
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import numpy_moe  # noqa: E402
from neonengine_b200 import synth  # noqa: E402


def wdict(W):
    return {k: getattr(W, k) for k in ("router_w", "router_b", "gate_up_blocks", "gate_up_scales", "gate_up_bias",
                                       "down_blocks", "down_scales", "down_bias")}


def save(name, hidden, W, k, logit_bias=None):
    out, idx, w, lg = numpy_moe.forward(hidden, W, logit_bias=logit_bias, k=k)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), hidden=hidden, out=out, idx=idx, w=w, logits=lg,
                        top_k=np.int32(k), logit_bias=np.zeros(0, np.float32) if logit_bias is None else logit_bias,
                        **W)
    print(name, out.shape, float(np.abs(out).max()))


def main():
    sh = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    W = synth.make_weights(sh, base_seed=7)
    hidden = synth.make_hidden(6, W, base_seed=7)
    save("small_seeded", hidden, wdict(W), 4)
    save("small_seeded_zipf", hidden, wdict(W), 4, synth.zipf_logit_bias(8))

    E, H, I, k = 4, 64, 64, 2
    one = synth.f32_to_bf16_bits(np.array([1.0], np.float32))[0]
    Wi = dict(router_w=np.zeros((E, H), np.uint16), router_b=np.zeros(E, np.uint16),
              gate_up_blocks=np.full((E, 2 * I, H // 2), 0x22, np.uint8),
              gate_up_scales=np.full((E, 2 * I, H // 32), 127, np.uint8),
              gate_up_bias=np.zeros((E, 2 * I), np.uint16),
              down_blocks=np.full((E, H, I // 2), 0x22, np.uint8),
              down_scales=np.full((E, H, I // 32), 127, np.uint8),
              down_bias=np.zeros((E, H), np.uint16))
    # distinct router rows so that routing is decided: logit_e = (e+1) * sum(x) * 2^-6
    for e in range(E):
        Wi["router_w"][e, :] = synth.f32_to_bf16_bits(np.full(H, (e + 1) / 64.0, np.float32))
    ones = np.full((2, H), one, np.uint16)
    save("integer_kat", ones, Wi, k)
    neg = synth.f32_to_bf16_bits(np.full((2, H), -1.0, np.float32))
    save("clamp_negative", neg, Wi, k)
    Wt = dict(Wi)
    Wt["router_w"] = np.zeros((E, H), np.uint16)
    save("all_ties", ones, Wt, k)


if __name__ == "__main__":
    main()
