"""Seeded synthetic inputs for the gpt-oss-shaped MoE layer.

Every tensor comes from its own ``numpy.random.Generator(PCG64(base_seed + tensor_id))``
so the CUDA path, the CPU oracle and every expert-parallel rank regenerate identical
bits.  Distributions follow the benchmark configuration text:

* hidden states           bf16  N(0, 1)                    [T, H]
* router weight / bias    bf16  N(0, 0.02)                 [E, H] / [E]
* expert nibbles          e2m1 codes uniform over 0..15    packed two per byte
* expert block scales     E8M0, exponent uniform integer in [-10, -4] (bytes 117..123)
* expert biases           bf16  N(0, 0.02)

Storage conventions shared by the C ABI, the kernels and the oracle:

* bf16 tensors are ``uint16`` arrays holding the raw bit pattern.
* MXFP4 blocks: ``uint8 [E, rows, cols/2]``; the LOW nibble of byte ``j`` is column
  ``2j``, the high nibble column ``2j+1``.  Code bits are ``s e e m``.
* Scales: ``uint8 [E, rows, cols/32]``, value ``2**(byte-127)``.
* gate_up rows are interleaved: even row ``2i`` is the gate ("x_glu") of intermediate
  channel ``i``, odd row ``2i+1`` is the linear half ("x_lin").

The reference engine (a Vulkan renderer) holds no generator or data format for this
path; these conventions are this library's own.
"""
from __future__ import annotations

import dataclasses

import numpy as np

TENSOR_IDS = {
    "hidden": 1, "router_w": 2, "router_b": 3,
    "gate_up_blocks": 4, "gate_up_scales": 5, "gate_up_bias": 6,
    "down_blocks": 7, "down_scales": 8, "down_bias": 9,
}

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as raw uint16 bits."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _rng(base_seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(base_seed + TENSOR_IDS[name]))


@dataclasses.dataclass
class MoeShape:
    hidden: int = 2880
    inter: int = 2880
    n_experts: int = 32
    top_k: int = 4
    swiglu_limit: float = 7.0
    swiglu_alpha: float = 1.702

    @property
    def expert_bytes(self) -> int:
        """Bytes of one expert: nibbles + scales + bf16 biases of gate_up and down."""
        H, I = self.hidden, self.inter
        gu = 2 * I * H // 2 + 2 * I * H // 32 + 2 * I * 2
        dn = H * I // 2 + H * I // 32 + H * 2
        return gu + dn

    @property
    def router_bytes(self) -> int:
        return self.n_experts * self.hidden * 2 + self.n_experts * 2

    @property
    def flops_per_pair(self) -> int:
        """Flops of one (token, expert) pair: gate_up plus down."""
        return 2 * 2 * self.inter * self.hidden + 2 * self.hidden * self.inter


@dataclasses.dataclass
class MoeWeights:
    shape: MoeShape
    router_w: np.ndarray         # uint16 [E, H]
    router_b: np.ndarray         # uint16 [E]
    gate_up_blocks: np.ndarray   # uint8 [E, 2I, H/2]
    gate_up_scales: np.ndarray   # uint8 [E, 2I, H/32]
    gate_up_bias: np.ndarray     # uint16 [E, 2I]
    down_blocks: np.ndarray      # uint8 [E, H, I/2]
    down_scales: np.ndarray      # uint8 [E, H, I/32]
    down_bias: np.ndarray        # uint16 [E, H]

    def slice_experts(self, lo: int, hi: int) -> "MoeWeights":
        """Expert-parallel shard: experts [lo, hi) with the full (replicated) router."""
        return MoeWeights(self.shape, self.router_w, self.router_b,
                          self.gate_up_blocks[lo:hi], self.gate_up_scales[lo:hi],
                          self.gate_up_bias[lo:hi], self.down_blocks[lo:hi],
                          self.down_scales[lo:hi], self.down_bias[lo:hi])


def make_weights(shape: MoeShape, base_seed: int = 0, experts: tuple[int, int] | None = None) -> MoeWeights:
    """Generate the layer's weights.  ``experts=(lo, hi)`` generates only that expert
    range (bit-identical to the same slice of a full generation) so that an
    expert-parallel rank never materialises other ranks' experts."""
    H, I, E = shape.hidden, shape.inter, shape.n_experts
    assert H % 32 == 0 and I % 32 == 0
    lo, hi = (0, E) if experts is None else experts

    def per_expert(name, fn):
        # one child stream per expert keeps a shard bit-identical to the full tensor
        base = np.random.SeedSequence(base_seed + TENSOR_IDS[name])
        kids = base.spawn(E)
        return np.stack([fn(np.random.Generator(np.random.PCG64(kids[e]))) for e in range(lo, hi)])

    router_w = f32_to_bf16_bits(_rng(base_seed, "router_w").normal(0.0, 0.02, (E, H)).astype(np.float32))
    router_b = f32_to_bf16_bits(_rng(base_seed, "router_b").normal(0.0, 0.02, (E,)).astype(np.float32))
    gub = per_expert("gate_up_blocks", lambda g: g.integers(0, 256, (2 * I, H // 2), dtype=np.uint8))
    gus = per_expert("gate_up_scales", lambda g: g.integers(117, 124, (2 * I, H // 32), dtype=np.uint8))
    gubias = per_expert("gate_up_bias", lambda g: f32_to_bf16_bits(g.normal(0.0, 0.02, (2 * I,)).astype(np.float32)))
    db = per_expert("down_blocks", lambda g: g.integers(0, 256, (H, I // 2), dtype=np.uint8))
    ds = per_expert("down_scales", lambda g: g.integers(117, 124, (H, I // 32), dtype=np.uint8))
    dbias = per_expert("down_bias", lambda g: f32_to_bf16_bits(g.normal(0.0, 0.02, (H,)).astype(np.float32)))
    return MoeWeights(shape, router_w, router_b, gub, gus, gubias, db, ds, dbias)


def zipf_logit_bias(n_experts: int, s: float = 1.1) -> np.ndarray:
    """Additive per-expert router bias that skews loads Zipf-like: ``-s*ln(e+1)``
    (the log of an unnormalised Zipf(s) mass; the constant is irrelevant to top-k and
    to a softmax over the selected logits)."""
    return (-s * np.log(np.arange(1, n_experts + 1, dtype=np.float64))).astype(np.float32)


def router_logits_f64(hidden_bits, weights: MoeWeights, logit_bias=None) -> np.ndarray:
    x = bf16_bits_to_f32(hidden_bits).astype(np.float64)
    w = bf16_bits_to_f32(weights.router_w).astype(np.float64)
    b = bf16_bits_to_f32(weights.router_b).astype(np.float64)
    lg = x @ w.T + b
    if logit_bias is not None:
        lg = lg + np.asarray(logit_bias, dtype=np.float64)
    return lg


def make_hidden(T: int, weights: MoeWeights, base_seed: int = 0, logit_bias=None,
                min_gap: float = 1e-4, stream: int = 0) -> np.ndarray:
    """bf16 N(0,1) hidden states [T, H] as uint16 bits.

    Routing indices must match bit-exactly between an fp32-accumulating GPU router and
    the fp64 oracle, which is only well defined when the five largest logits of a token
    are separated by more than accumulation noise.  Tokens whose adjacent gaps among the
    top ``k+1`` logits fall under ``min_gap`` are redrawn from a deterministic
    per-token substream until they clear it.  ``stream`` selects independent batches
    (bench steps, expert-parallel ranks)."""
    H = weights.shape.hidden
    k = weights.shape.top_k
    seq = np.random.SeedSequence([base_seed + TENSOR_IDS["hidden"], stream])
    g = np.random.Generator(np.random.PCG64(seq))
    hid = f32_to_bf16_bits(g.normal(0.0, 1.0, (T, H)).astype(np.float32))
    if min_gap <= 0:
        return hid
    for attempt in range(1, 32):
        lg = router_logits_f64(hid, weights, logit_bias)
        top = -np.sort(-lg, axis=1)[:, :k + 1]
        bad = np.nonzero((top[:, :-1] - top[:, 1:]).min(axis=1) < min_gap)[0]
        if bad.size == 0:
            return hid
        for t in bad:
            sub = np.random.Generator(np.random.PCG64(
                np.random.SeedSequence([base_seed + TENSOR_IDS["hidden"], stream, int(t), attempt])))
            hid[t] = f32_to_bf16_bits(sub.normal(0.0, 1.0, (H,)).astype(np.float32))
    raise RuntimeError("could not separate router logits")


def dequant_mxfp4(blocks: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """Exact fp32 dequantisation of [..., rows, cols/2] nibbles with [..., rows, cols/32] scales."""
    lo = E2M1_VALUES[blocks & 0x0F]
    hi = E2M1_VALUES[blocks >> 4]
    vals = np.stack([lo, hi], axis=-1).reshape(*blocks.shape[:-1], blocks.shape[-1] * 2)
    sc = np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127).astype(np.float32)
    return vals * np.repeat(sc, 32, axis=-1)
