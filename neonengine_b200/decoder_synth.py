"""Seeded synthetic weights and caches for the gpt-oss-shaped decoder stack.

Distributions: projection, embedding and bias tensors N(0, 0.02); norm weights
1 + N(0, 0.1); per-head sink logits N(0, 1); cached keys and values N(0, 1); all stored
as bf16 bit patterns.  MoE tensors come from :func:`neonengine_b200.synth.make_weights`.
"""
from __future__ import annotations

import dataclasses

import numpy as np

from .synth import MoeShape, MoeWeights, f32_to_bf16_bits, make_weights


@dataclasses.dataclass
class DecoderShape:
    n_layers: int = 24
    hidden: int = 2880
    n_q_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 64
    vocab: int = 201088
    window: int = 128
    rope_theta: float = 150000.0
    rope_factor: float = 32.0
    rope_orig_ctx: float = 4096.0
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rms_eps: float = 1e-5
    moe: MoeShape = dataclasses.field(default_factory=MoeShape)

    @property
    def qkv_rows(self) -> int:
        return (self.n_q_heads + 2 * self.n_kv_heads) * self.head_dim

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim


@dataclasses.dataclass
class AttentionWeights:
    ln1: np.ndarray    # uint16 [H]
    wqkv: np.ndarray   # uint16 [qkv_rows, H]
    bqkv: np.ndarray   # uint16 [qkv_rows]
    sinks: np.ndarray  # uint16 [n_q_heads]
    wo: np.ndarray     # uint16 [H, q_dim]
    bo: np.ndarray     # uint16 [H]
    ln2: np.ndarray    # uint16 [H]


@dataclasses.dataclass
class DecoderWeights:
    shape: DecoderShape
    embed: np.ndarray       # uint16 [vocab, H]
    unembed: np.ndarray     # uint16 [vocab, H]
    final_norm: np.ndarray  # uint16 [H]
    attention: list         # AttentionWeights per layer
    moe: list               # MoeWeights per layer


def _bits(g: np.random.Generator, mean: float, std: float, shape) -> np.ndarray:
    return f32_to_bf16_bits((mean + std * g.standard_normal(shape, dtype=np.float32)).astype(np.float32))


def make_attention_weights(shape: DecoderShape, layer: int, base_seed: int = 0) -> AttentionWeights:
    g = np.random.Generator(np.random.PCG64(np.random.SeedSequence([base_seed, 7001, layer])))
    H = shape.hidden
    return AttentionWeights(
        ln1=_bits(g, 1.0, 0.1, (H,)),
        wqkv=_bits(g, 0.0, 0.02, (shape.qkv_rows, H)),
        bqkv=_bits(g, 0.0, 0.02, (shape.qkv_rows,)),
        sinks=_bits(g, 0.0, 1.0, (shape.n_q_heads,)),
        wo=_bits(g, 0.0, 0.02, (H, shape.q_dim)),
        bo=_bits(g, 0.0, 0.02, (H,)),
        ln2=_bits(g, 1.0, 0.1, (H,)),
    )


def make_decoder_weights(shape: DecoderShape, base_seed: int = 0, share_moe: bool = False) -> DecoderWeights:
    """All tensors on the host (meant for test-sized shapes).  ``share_moe`` reuses layer 0's
    expert tensors in every layer (the routers still differ) to bound generation time."""
    assert shape.moe.hidden == shape.hidden
    g = np.random.Generator(np.random.PCG64(np.random.SeedSequence([base_seed, 7000])))
    embed = _bits(g, 0.0, 0.02, (shape.vocab, shape.hidden))
    unembed = _bits(g, 0.0, 0.02, (shape.vocab, shape.hidden))
    final_norm = _bits(g, 1.0, 0.1, (shape.hidden,))
    attention = [make_attention_weights(shape, l, base_seed) for l in range(shape.n_layers)]
    moe = []
    for l in range(shape.n_layers):
        if share_moe and l > 0:
            w0 = moe[0]
            r = make_weights(dataclasses.replace(shape.moe, inter=32), base_seed + 1000 * (l + 1))  # router only
            moe.append(MoeWeights(shape.moe, r.router_w, r.router_b, w0.gate_up_blocks, w0.gate_up_scales,
                                  w0.gate_up_bias, w0.down_blocks, w0.down_scales, w0.down_bias))
        else:
            moe.append(make_weights(shape.moe, base_seed + 1000 * (l + 1)))
    return DecoderWeights(shape, embed, unembed, final_norm, attention, moe)


def make_kv(shape: DecoderShape, layer: int, batch: int, n_pos: int, base_seed: int = 0):
    """Cached keys and values of one layer: two uint16 [batch, n_pos, n_kv_heads, head_dim]."""
    g = np.random.Generator(np.random.PCG64(np.random.SeedSequence([base_seed, 7002, layer])))
    dims = (batch, n_pos, shape.n_kv_heads, shape.head_dim)
    return _bits(g, 0.0, 1.0, dims), _bits(g, 0.0, 1.0, dims)
