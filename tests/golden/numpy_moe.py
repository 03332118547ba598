"""Independent numpy float64 restatement of the MoE layer math, used to generate and to
check the golden vectors.  It shares no code with oracle/moe_oracle.c: the dequantiser,
the top-k and the SwiGLU are written again here from the benchmark configuration text
(the nominal reference engine has no implementation of this path to import)."""
import numpy as np

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def bf16(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def deq(blocks, scales):
    lo, hi = E2M1[blocks & 15], E2M1[blocks >> 4]
    v = np.empty(blocks.shape[:-1] + (blocks.shape[-1] * 2,), np.float64)
    v[..., 0::2], v[..., 1::2] = lo, hi
    return v * np.repeat(np.exp2(scales.astype(np.float64) - 127.0), 32, axis=-1)


def route(hidden, router_w, router_b, k, logit_bias=None):
    lg = bf16(hidden) @ bf16(router_w).T + bf16(router_b)
    if logit_bias is not None:
        lg = lg + np.asarray(logit_bias, np.float64)
    lg = lg.astype(np.float32)
    T, E = lg.shape
    idx = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    for t in range(T):
        order = np.lexsort((np.arange(E), -lg[t].astype(np.float64)))[:k]  # by -logit, then id
        idx[t] = order
        sel = lg[t, order].astype(np.float64)
        p = np.exp(sel - sel.max())
        w[t] = (p / p.sum()).astype(np.float32)
    return idx, w, lg


def forward(hidden, W, logit_bias=None, limit=7.0, alpha=1.702, k=4):
    """W: dict with router_w, router_b, gate_up_blocks/scales/bias, down_blocks/scales/bias."""
    idx, w, lg = route(hidden, W["router_w"], W["router_b"], k, logit_bias)
    x = bf16(hidden)
    T, H = x.shape
    out = np.zeros((T, H), np.float64)
    for t in range(T):
        for s in range(k):
            e = int(idx[t, s])
            gu = deq(W["gate_up_blocks"][e], W["gate_up_scales"][e]) @ x[t] + bf16(W["gate_up_bias"][e])
            g = np.minimum(gu[0::2], limit)
            lin = np.clip(gu[1::2], -limit, limit)
            a = g * (1.0 / (1.0 + np.exp(-alpha * g))) * (lin + 1.0)
            y = deq(W["down_blocks"][e], W["down_scales"][e]) @ a + bf16(W["down_bias"][e])
            out[t] += np.float64(w[t, s]) * y
    return out.astype(np.float32), idx, w, lg
