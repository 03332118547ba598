"""ctypes front end of the CPU oracle (``moe_oracle.c``).

Test infrastructure: only tests, the smoke check and the benchmark's CPU-baseline leg
import this package.  Parity with the nominal reference is unpinned (it has no such
path); the oracle restates the benchmark configuration's layer math in fp64.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "moe_oracle.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_SO = os.path.join(_OUT_DIR, "libmoe_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (AVX2 baseline so the file runs on any recent host)."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    os.makedirs(_OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c11",
           _SRC, "-o", _SO, "-lm"]
    subprocess.run(cmd, check=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a, ty=ctypes.c_void_p):
    return None if a is None else a.ctypes.data_as(ty)


def n_threads() -> int:
    return len(os.sched_getaffinity(0))


def route(hidden, router_w, router_b, top_k, logit_bias=None, want_logits=False):
    T, H = hidden.shape
    E = router_w.shape[0]
    hidden = np.ascontiguousarray(hidden, np.uint16)
    idx = np.empty((T, top_k), np.int32)
    w = np.empty((T, top_k), np.float32)
    logits = np.empty((T, E), np.float32) if want_logits else None
    lb = None if logit_bias is None else np.ascontiguousarray(logit_bias, np.float32)
    lib().oracle_route(_p(hidden), _p(np.ascontiguousarray(router_w)), _p(np.ascontiguousarray(router_b)),
                       _p(lb), T, H, E, top_k, _p(idx), _p(w), _p(logits))
    return (idx, w, logits) if want_logits else (idx, w)


def dispatch(idx, n_experts):
    T, k = idx.shape
    idx = np.ascontiguousarray(idx, np.int32)
    count = np.empty(n_experts, np.int32)
    offset = np.empty(n_experts + 1, np.int32)
    perm = np.empty(T * k, np.int32)
    inv = np.empty(T * k, np.int32)
    lib().oracle_dispatch(_p(idx), T, k, n_experts, _p(count), _p(offset), _p(perm), _p(inv))
    return count, offset, perm, inv


def experts(hidden, idx, w, weights, tokens=None, quant_act=False, e_lo=0):
    """Expert products + SwiGLU + combine.  ``weights`` holds experts [e_lo, e_lo+E_local)."""
    T, H = hidden.shape
    k = idx.shape[1]
    I = weights.down_blocks.shape[2] * 2
    E_local = weights.gate_up_blocks.shape[0]
    sh = weights.shape
    hidden = np.ascontiguousarray(hidden, np.uint16)
    idx = np.ascontiguousarray(idx, np.int32)
    w = np.ascontiguousarray(w, np.float32)
    tok = None if tokens is None else np.ascontiguousarray(tokens, np.int32)
    n = T if tok is None else tok.size
    out = np.empty((n, H), np.float32)
    c = np.ascontiguousarray
    lib().oracle_experts(_p(hidden), _p(idx), _p(w), T, H, I, k, e_lo, E_local,
                         _p(c(weights.gate_up_blocks)), _p(c(weights.gate_up_scales)), _p(c(weights.gate_up_bias)),
                         _p(c(weights.down_blocks)), _p(c(weights.down_scales)), _p(c(weights.down_bias)),
                         ctypes.c_float(sh.swiglu_limit), ctypes.c_float(sh.swiglu_alpha),
                         _p(tok), n, int(quant_act), _p(out))
    return out


def moe_forward(hidden, weights, logit_bias=None, tokens=None, quant_act=False):
    """Whole layer: returns (out[T or len(tokens), H] fp32, idx[T,k], w[T,k])."""
    idx, w = route(hidden, weights.router_w, weights.router_b, weights.shape.top_k, logit_bias)
    out = experts(hidden, idx, w, weights, tokens=tokens, quant_act=quant_act)
    return out, idx, w


def swiglu(gu, limit=7.0, alpha=1.702):
    gu = np.ascontiguousarray(gu, np.float64)
    a = np.empty(gu.size // 2, np.float64)
    lib().oracle_swiglu(_p(gu), a.size, ctypes.c_float(limit), ctypes.c_float(alpha), _p(a))
    return a
