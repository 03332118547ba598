"""CPU restatement of the decoder stack around the MoE layer (numpy, float64 arithmetic).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU-baseline leg of
the benchmark, never by the product path.  PARITY UNPINNED: the reference engine
(NeonEngine) holds no language-model code, golden vectors or fixtures for this path, so
this file restates the published algorithms (RMSNorm; rotary embedding with YaRN
"NTK-by-parts" frequency blending, Peng et al. 2023, section 3.2-3.4; grouped-query
softmax attention with a per-head sink logit in the denominator and an optional sliding
window; residual connections) under the conventions written in include/neon_decoder.h.

Rounding points mirror the interface: normalised activations, attention outputs and
cached K/V are rounded to bf16 (nearest even); everything else is float64 here (fp32 on
the GPU).
"""
from __future__ import annotations

import math

import numpy as np

from neonengine_b200.synth import bf16_bits_to_f32, f32_to_bf16_bits


def _f(bits) -> np.ndarray:
    return bf16_bits_to_f32(np.asarray(bits)).astype(np.float64)


def _round_bf16(x) -> np.ndarray:
    """float64 -> bf16 bit patterns (through fp32, round to nearest even)."""
    return f32_to_bf16_bits(np.asarray(x, np.float64).astype(np.float32))


def yarn_inv_freq(shape):
    """Returns (inv_freq float32 [head_dim/2], mscale)."""
    d = shape.head_dim
    theta, factor = float(shape.rope_theta), float(shape.rope_factor)

    def corr_dim(n_rot):
        return d * math.log(shape.rope_orig_ctx / (n_rot * 2.0 * math.pi)) / (2.0 * math.log(theta))

    inv = np.empty(d // 2, np.float64)
    if factor > 1.0:
        low = max(math.floor(corr_dim(shape.rope_beta_fast)), 0.0)
        high = min(math.ceil(corr_dim(shape.rope_beta_slow)), float(d - 1))
        if high == low:
            high += 0.001
    for i in range(d // 2):
        freq = theta ** (2.0 * i / d)
        v = 1.0 / freq
        if factor > 1.0:
            ramp = min(max((i - low) / (high - low), 0.0), 1.0)
            keep = 1.0 - ramp
            v = (1.0 / (factor * freq)) * (1.0 - keep) + (1.0 / freq) * keep
        inv[i] = v
    mscale = 0.1 * math.log(factor) + 1.0 if factor > 1.0 else 1.0
    return inv.astype(np.float32), float(np.float32(mscale))


def rmsnorm(x, w_bits, eps) -> np.ndarray:
    """x float [B, H] -> bf16 bits [B, H]."""
    x = np.asarray(x, np.float64)
    r = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return _round_bf16(x * r * _f(w_bits))


def linear(x_bits, w_bits, b_bits=None) -> np.ndarray:
    """bf16 activations [B, K] times bf16 weights [rows, K] (+ bf16 bias) in float64."""
    y = _f(x_bits) @ _f(w_bits).T
    return y if b_bits is None else y + _f(b_bits)


def rope(v, pos, inv_freq, mscale) -> np.ndarray:
    """v float [B, heads, D]; element i pairs with i + D/2."""
    v = np.asarray(v, np.float64)
    half = v.shape[-1] // 2
    # the kernel forms the angle in fp32 (position * inv_freq) before sin/cos
    ang = (np.asarray(pos, np.float32)[:, None] * inv_freq[None, :].astype(np.float32)).astype(np.float64)
    c = (np.cos(ang) * mscale)[:, None, :]
    s = (np.sin(ang) * mscale)[:, None, :]
    a, b = v[..., :half], v[..., half:]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def attention(q, kcache_bits, vcache_bits, pos, sinks_bits, window) -> np.ndarray:
    """q float [B, nq, D] (rotated); caches bf16 bits [B, ctx, nkv, D] already holding the
    new token at pos[b]; returns float64 [B, nq*D] before bf16 rounding."""
    q = np.asarray(q, np.float64)
    B, nq, D = q.shape
    nkv = kcache_bits.shape[2]
    G = nq // nkv
    sinks = _f(sinks_bits)
    out = np.zeros((B, nq, D))
    for b in range(B):
        p = int(pos[b])
        lo = max(0, p - window + 1) if window > 0 else 0
        k = _f(kcache_bits[b, lo:p + 1])  # [n, nkv, D]
        v = _f(vcache_bits[b, lo:p + 1])
        for h in range(nq):
            s = k[:, h // G, :] @ q[b, h] / math.sqrt(D)
            m = max(s.max(), sinks[h])
            e = np.exp(s - m)
            out[b, h] = (e[:, None] * v[:, h // G, :]).sum(0) / (e.sum() + math.exp(sinks[h] - m))
    return out.reshape(B, nq * D)


def decoder_step(weights, kcaches, vcaches, tokens, positions, moe_fn, n_layers=None, moe_in_override=None):
    """One decode step.  kcaches/vcaches: per-layer uint16 [B, ctx, nkv, D] arrays, updated in
    place at positions[b].  moe_fn(layer, xn_bits) -> float [B, H] runs the MoE layer.
    moe_in_override: optional {layer: bf16 bits} replacing the MoE input of that layer (lets a
    test feed the device's own bit pattern so that routing is compared on equal inputs).
    Returns a dict with the last layer's intermediates, the residual stream and the logits."""
    sh = weights.shape
    inv_freq, mscale = yarn_inv_freq(sh)
    B = len(tokens)
    nq, nkv, D = sh.n_q_heads, sh.n_kv_heads, sh.head_dim
    x = _f(weights.embed[np.asarray(tokens)])
    r = {}
    L = sh.n_layers if n_layers is None else n_layers
    for l in range(L):
        a = weights.attention[l]
        xn = rmsnorm(x, a.ln1, sh.rms_eps)
        qkv = linear(xn, a.wqkv, a.bqkv)
        q = rope(qkv[:, :nq * D].reshape(B, nq, D), positions, inv_freq, mscale)
        k = rope(qkv[:, nq * D:(nq + nkv) * D].reshape(B, nkv, D), positions, inv_freq, mscale)
        v = qkv[:, (nq + nkv) * D:].reshape(B, nkv, D)
        for b in range(B):
            kcaches[l][b, positions[b]] = _round_bf16(k[b])
            vcaches[l][b, positions[b]] = _round_bf16(v[b])
        window = sh.window if (sh.window > 0 and l % 2 == 0) else 0
        att = _round_bf16(attention(q, kcaches[l], vcaches[l], positions, a.sinks, window))
        x = x + linear(att, a.wo, a.bo)
        xn2 = rmsnorm(x, a.ln2, sh.rms_eps)
        if moe_in_override is not None and l in moe_in_override:
            xn2 = np.asarray(moe_in_override[l])
        moe_out = np.asarray(moe_fn(l, xn2), np.float64)
        r.update(q=q, qkv_kv=qkv[:, nq * D:], attn=att, moe_in=xn2, moe_out=moe_out, x_mid=x)
        x = x + moe_out
    r["x"] = x
    xn = rmsnorm(x, weights.final_norm, sh.rms_eps)
    r["xn"] = xn
    r["logits"] = linear(xn, weights.unembed)
    r["next"] = np.argmax(r["logits"], axis=-1).astype(np.int32)
    return r
