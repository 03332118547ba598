"""Python host mirror of the decoder stack's C ABI (include/neon_decoder.h).

Shaped like the engine's compute systems (NeonEngine/src/water_physics.hpp:66): the
constructor owns the device buffers, weights are uploaded once, ``step`` enqueues one
decode step on a stream, errors become ``RuntimeError``.  torch only owns device memory and
streams; every kernel runs inside ``libneon_moe.so``.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .decoder_synth import AttentionWeights, DecoderShape, DecoderWeights
from .synth import MoeWeights


def _ptrs(arrays):
    """Addresses of numpy arrays (host) or torch CUDA tensors (device); one residency per call."""
    on_device = [hasattr(a, "is_cuda") for a in arrays]
    assert all(on_device) or not any(on_device), "mix of host and device tensors"
    if all(on_device):
        assert all(a.is_cuda and a.is_contiguous() for a in arrays)
        return [ctypes.c_void_p(a.data_ptr()) for a in arrays], 1, arrays
    keep = [np.ascontiguousarray(a) for a in arrays]
    return [ctypes.c_void_p(a.ctypes.data) for a in keep], 0, keep


class DecoderSystem:
    def __init__(self, shape: DecoderShape, max_batch: int, max_ctx: int, device: int = 0):
        self._lib = _lib.load()
        self.shape, self.max_batch, self.max_ctx, self.device = shape, int(max_batch), int(max_ctx), int(device)
        m = shape.moe
        cfg = _lib.NeonDecoderConfig(shape.n_layers, shape.hidden, shape.n_q_heads, shape.n_kv_heads, shape.head_dim,
                                     shape.vocab, self.max_batch, self.max_ctx, shape.window, shape.rope_theta,
                                     shape.rope_factor, shape.rope_orig_ctx, shape.rope_beta_fast, shape.rope_beta_slow,
                                     shape.rms_eps, m.inter, m.n_experts, m.top_k, m.swiglu_limit, m.swiglu_alpha,
                                     self.device)
        handle = ctypes.c_void_p()
        rc = self._lib.neon_decoder_create(ctypes.byref(cfg), ctypes.byref(handle))
        if rc != 0:
            raise RuntimeError(f"neon_decoder_create failed ({rc}): {self._lib.neon_decoder_last_error(None).decode()}")
        self._h = handle

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc}): {self._lib.neon_decoder_last_error(self._h).decode()}")

    # -- weights -------------------------------------------------------------------------
    def set_embeddings(self, embed, unembed, final_norm) -> None:
        p, dev, _keep = _ptrs([embed, unembed, final_norm])
        self._check(self._lib.neon_decoder_set_embeddings(self._h, *p, dev), "neon_decoder_set_embeddings")

    def set_attention(self, layer: int, a: AttentionWeights) -> None:
        p, dev, _keep = _ptrs([a.ln1, a.wqkv, a.bqkv, a.sinks, a.wo, a.bo, a.ln2])
        self._check(self._lib.neon_decoder_set_attention(self._h, layer, *p, dev), "neon_decoder_set_attention")

    def set_moe(self, layer: int, w: MoeWeights) -> None:
        p, dev, _keep = _ptrs([w.router_w, w.router_b, w.gate_up_blocks, w.gate_up_scales, w.gate_up_bias,
                               w.down_blocks, w.down_scales, w.down_bias])
        self._check(self._lib.neon_decoder_set_moe(self._h, layer, *p, dev), "neon_decoder_set_moe")

    def set_weights(self, w: DecoderWeights) -> None:
        self.set_embeddings(w.embed, w.unembed, w.final_norm)
        for l in range(self.shape.n_layers):
            self.set_attention(l, w.attention[l])
            self.set_moe(l, w.moe[l])

    def load_kv(self, layer: int, k, v) -> None:
        """k, v: bf16 bit patterns [batch, n_pos, n_kv_heads, head_dim] (keys already rotated)."""
        p, dev, _keep = _ptrs([k, v])
        self._check(self._lib.neon_decoder_load_kv(self._h, layer, *p, int(k.shape[0]), int(k.shape[1]), dev),
                    "neon_decoder_load_kv")

    # -- execution -----------------------------------------------------------------------
    def step(self, tokens, positions, logits=None, next_tokens=None, stream=None):
        """One decode step over device tensors: ``tokens``/``positions`` torch int32 [B];
        optional ``logits`` fp32 [B, vocab] and ``next_tokens`` int32 [B] outputs."""
        import torch
        assert tokens.is_cuda and positions.is_cuda and tokens.dtype == torch.int32 and positions.dtype == torch.int32
        st = torch.cuda.current_stream(tokens.device) if stream is None else stream
        self._check(self._lib.neon_decoder_step(
            self._h, ctypes.c_void_p(tokens.data_ptr()), ctypes.c_void_p(positions.data_ptr()), int(tokens.shape[0]),
            None if logits is None else ctypes.c_void_p(logits.data_ptr()),
            None if next_tokens is None else ctypes.c_void_p(next_tokens.data_ptr()),
            ctypes.c_void_p(st.cuda_stream)), "neon_decoder_step")

    def step_host(self, tokens: np.ndarray, positions: np.ndarray, stream=None) -> np.ndarray:
        """One decode step from host arrays; returns the next token of every sequence."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        positions = np.ascontiguousarray(positions, np.int32)
        nxt = np.empty(tokens.shape[0], np.int32)
        self.step_host_ptr(tokens.ctypes.data, positions.ctypes.data, tokens.shape[0], nxt.ctypes.data, stream)
        return nxt

    def step_host_ptr(self, tokens_ptr: int, positions_ptr: int, batch: int, next_ptr: int, stream=None) -> None:
        st = None if stream is None else ctypes.c_void_p(stream.cuda_stream)
        self._check(self._lib.neon_decoder_step_host(self._h, ctypes.c_void_p(tokens_ptr), ctypes.c_void_p(positions_ptr),
                                                     int(batch), ctypes.c_void_p(next_ptr), st), "neon_decoder_step_host")

    # -- inspection ----------------------------------------------------------------------
    _BUFFERS = {"x": (np.float32, "H"), "xn": (np.uint16, "H"), "moe_in": (np.uint16, "H"), "moe_out": (np.float32, "H"),
                "qkv": (np.float32, "QKV"), "attn": (np.uint16, "QD"), "logits": (np.float32, "V")}

    def read(self, name: str, batch: int | None = None) -> np.ndarray:
        if name == "inv_freq":
            out = np.empty(32, np.float32)
        else:
            dtype, dim = self._BUFFERS[name]
            cols = {"H": self.shape.hidden, "QKV": self.shape.qkv_rows, "QD": self.shape.q_dim, "V": self.shape.vocab}[dim]
            out = np.empty((self.max_batch if batch is None else batch, cols), dtype)
        self._check(self._lib.neon_decoder_read(self._h, name.encode(), ctypes.c_void_p(out.ctypes.data), out.nbytes),
                    "neon_decoder_read")
        return out

    def set_option(self, name: str, value: int) -> None:
        self._check(self._lib.neon_decoder_set_option(self._h, name.encode(), int(value)), "neon_decoder_set_option")

    def launch_count(self) -> int:
        return int(self._lib.neon_decoder_launch_count(self._h))

    def step_bytes(self, positions: np.ndarray):
        """(dense weight bytes, K/V bytes, MoE expert bytes) the last step had to read at least."""
        positions = np.ascontiguousarray(positions, np.int32)
        out = (ctypes.c_double * 3)()
        self._check(self._lib.neon_decoder_step_bytes(self._h, ctypes.c_void_p(positions.ctypes.data), positions.shape[0], out),
                    "neon_decoder_step_bytes")
        return tuple(out)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.neon_decoder_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
