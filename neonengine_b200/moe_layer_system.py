"""Python mirror of the C++ ``lve::MoeLayerSystem`` wrapper (include/lve_moe_layer_system.hpp).

Same shape as the engine's compute systems (NeonEngine/src/water_physics.hpp:66,
NeonEngine/src/raytracing_system.hpp:79): the constructor creates the layer and uploads
the weights, ``run`` enqueues one pass on a stream, a non-zero status becomes a
``RuntimeError`` (the C++ wrapper throws ``std::runtime_error``).  torch is used only to
own device memory and streams; all compute happens inside ``libneon_moe.so``.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .synth import MoeShape, MoeWeights


class MoeLayerSystem:
    def __init__(self, shape: MoeShape, weights: MoeWeights | None, max_tokens: int, device: int = 0,
                 ep_rank: int = 0, ep_size: int = 1):
        self._lib = _lib.load()
        self.shape = shape
        self.max_tokens = int(max_tokens)
        self.device = int(device)
        self.ep_rank, self.ep_size = int(ep_rank), int(ep_size)
        cfg = _lib.NeonMoeConfig(shape.hidden, shape.inter, shape.n_experts, shape.top_k,
                                 shape.swiglu_limit, shape.swiglu_alpha, self.max_tokens,
                                 self.ep_rank, self.ep_size, self.device)
        handle = ctypes.c_void_p()
        rc = self._lib.neon_moe_create(ctypes.byref(cfg), ctypes.byref(handle))
        if rc != 0:
            raise RuntimeError(f"neon_moe_create failed ({rc}): {self._lib.neon_moe_last_error(None).decode()}")
        self._h = handle
        if weights is not None:  # None: weights come from a file (load_weights_file)
            self.set_weights(weights)

    # -- helpers -------------------------------------------------------------------------
    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc}): {self._lib.neon_moe_last_error(self._h).decode()}")

    @staticmethod
    def _np_ptr(a):
        return None if a is None else ctypes.c_void_p(a.ctypes.data)

    def set_weights(self, w: MoeWeights) -> None:
        arrs = [np.ascontiguousarray(a) for a in (w.router_w, w.router_b, w.gate_up_blocks, w.gate_up_scales,
                                                  w.gate_up_bias, w.down_blocks, w.down_scales, w.down_bias)]
        self._check(self._lib.neon_moe_set_weights(self._h, *[self._np_ptr(a) for a in arrs], 0), "neon_moe_set_weights")

    def save_weights(self, path: str) -> None:
        """Writes the tensor-core layout as it sits in HBM ("tiled" weight file)."""
        self._check(self._lib.neon_moe_save_weights(self._h, str(path).encode()), "neon_moe_save_weights")

    def load_weights_file(self, path: str) -> None:
        """Loads a raw or tiled weight file (see include/neon_moe.h)."""
        self._check(self._lib.neon_moe_load_weights_file(self._h, str(path).encode()), "neon_moe_load_weights_file")

    # -- device path ---------------------------------------------------------------------
    def run(self, hidden, logit_bias=None, out=None, want_routing=False, stream=None):
        """One pass over device tensors.  ``hidden``: torch bf16 (or int16/uint16 bit view)
        [T, H] on this layer's GPU; returns fp32 [T, H] (and idx, w when ``want_routing``)."""
        import torch
        T = hidden.shape[0]
        assert hidden.is_cuda and hidden.is_contiguous() and hidden.element_size() == 2
        dev = hidden.device
        if out is None:
            out = torch.empty((T, self.shape.hidden), dtype=torch.float32, device=dev)
        idx = w = None
        if want_routing:
            idx = torch.empty((T, self.shape.top_k), dtype=torch.int32, device=dev)
            w = torch.empty((T, self.shape.top_k), dtype=torch.float32, device=dev)
        st = (stream or torch.cuda.current_stream(dev)).cuda_stream
        rc = self._lib.neon_moe_forward(self._h, hidden.data_ptr(), T,
                                        None if logit_bias is None else logit_bias.data_ptr(),
                                        out.data_ptr(), None if idx is None else idx.data_ptr(),
                                        None if w is None else w.data_ptr(), st)
        self._check(rc, "neon_moe_forward")
        return (out, idx, w) if want_routing else out

    def run_static(self, hidden, logit_bias=None, out=None, want_routing=False, stream=None):
        """Same pass as ``run`` through ``neon_moe_forward_static``: the intermediates live
        in the library's built-in 2 MiB device array instead of this handle's workspaces, so
        the call allocates nothing (``out`` and the routing tensors are the caller's; pass
        them in to avoid even torch's allocator).  Small batches only (T <= 22 at the
        gpt-oss shapes); calls that can overlap on one GPU must be ordered by the caller."""
        import torch
        T = hidden.shape[0]
        assert hidden.is_cuda and hidden.is_contiguous() and hidden.element_size() == 2
        dev = hidden.device
        if out is None:
            out = torch.empty((T, self.shape.hidden), dtype=torch.float32, device=dev)
        idx = w = None
        if want_routing:
            idx = torch.empty((T, self.shape.top_k), dtype=torch.int32, device=dev)
            w = torch.empty((T, self.shape.top_k), dtype=torch.float32, device=dev)
        st = (stream or torch.cuda.current_stream(dev)).cuda_stream
        rc = self._lib.neon_moe_forward_static(self._h, hidden.data_ptr(), T,
                                               None if logit_bias is None else logit_bias.data_ptr(),
                                               out.data_ptr(), None if idx is None else idx.data_ptr(),
                                               None if w is None else w.data_ptr(), st)
        if rc != 0:
            raise RuntimeError(f"neon_moe_forward_static failed ({rc}): {self._lib.neon_moe_last_error(None).decode()}")
        return (out, idx, w) if want_routing else out

    # -- expert parallelism --------------------------------------------------------------
    @staticmethod
    def ep_unique_id() -> bytes:
        """128-byte NCCL id; rank 0 creates it and passes it to the other ranks."""
        lib = _lib.load()
        buf = ctypes.create_string_buffer(128)
        rc = lib.neon_moe_ep_unique_id(buf)
        if rc != 0:
            raise RuntimeError(f"neon_moe_ep_unique_id failed ({rc}): {lib.neon_moe_last_error(None).decode()}")
        return buf.raw

    def ep_init(self, unique_id: bytes) -> None:
        """Collective: every rank of the expert-parallel group calls it with the same id."""
        assert len(unique_id) == 128
        self._check(self._lib.neon_moe_ep_init(self._h, ctypes.c_char_p(unique_id)), "neon_moe_ep_init")

    def ep_enable_peer_stores(self, all_gather_object) -> bool:
        """Collective: maps every peer's receive buffers (CUDA IPC) and, when that worked on EVERY rank,
        switches both exchanges to this library's own stores over NVLink.  ``all_gather_object(obj)`` must
        return the list of every rank's ``obj`` in rank order (e.g. a wrapper of
        ``torch.distributed.all_gather_object``).  Returns whether peer stores are in use."""
        buf = ctypes.create_string_buffer(128)
        ok = self._lib.neon_moe_ep_peer_export(self._h, buf) == 0
        handles = all_gather_object(buf.raw if ok else None)
        ok = ok and all(x is not None for x in handles)
        if ok:
            ok = self._lib.neon_moe_ep_peer_import(self._h, ctypes.c_char_p(b"".join(handles))) == 0
        ok = all(all_gather_object(bool(ok)))
        self.set_option("ep_peer", 1 if ok else 0)
        return ok

    def run_ep(self, hidden, logit_bias=None, out=None, want_routing=False, stream=None):
        """Expert-parallel pass over this rank's tokens (collective across the group)."""
        import torch
        T = hidden.shape[0]
        assert hidden.is_cuda and hidden.is_contiguous() and hidden.element_size() == 2
        dev = hidden.device
        if out is None:
            out = torch.empty((T, self.shape.hidden), dtype=torch.float32, device=dev)
        idx = w = None
        if want_routing:
            idx = torch.empty((T, self.shape.top_k), dtype=torch.int32, device=dev)
            w = torch.empty((T, self.shape.top_k), dtype=torch.float32, device=dev)
        st = (stream or torch.cuda.current_stream(dev)).cuda_stream
        rc = self._lib.neon_moe_forward_ep(self._h, hidden.data_ptr(), T,
                                           None if logit_bias is None else logit_bias.data_ptr(),
                                           out.data_ptr(), None if idx is None else idx.data_ptr(),
                                           None if w is None else w.data_ptr(), st)
        self._check(rc, "neon_moe_forward_ep")
        return (out, idx, w) if want_routing else out

    def ep_times(self):
        """Device times (ms) of the last expert-parallel pass and the rows this rank received."""
        ms = (ctypes.c_double * 5)()
        rows = ctypes.c_int(0)
        self._check(self._lib.neon_moe_ep_times(self._h, ms, ctypes.byref(rows)), "neon_moe_ep_times")
        names = ("route_pack", "dispatch_a2a", "experts", "combine_a2a", "combine")
        return dict(zip(names, list(ms))), rows.value

    # -- host path -----------------------------------------------------------------------
    def run_host(self, hidden: np.ndarray, logit_bias: np.ndarray | None = None, out: np.ndarray | None = None,
                 want_routing: bool = False):
        """One pass over HOST arrays (uint16 bf16 bits in, fp32 out); copies happen inside."""
        hidden = np.ascontiguousarray(hidden, np.uint16)
        T = hidden.shape[0]
        if out is None:
            out = np.empty((T, self.shape.hidden), np.float32)
        lb = None if logit_bias is None else np.ascontiguousarray(logit_bias, np.float32)
        idx = np.empty((T, self.shape.top_k), np.int32) if want_routing else None
        w = np.empty((T, self.shape.top_k), np.float32) if want_routing else None
        rc = self._lib.neon_moe_forward_host(self._h, self._np_ptr(hidden), T, self._np_ptr(lb), self._np_ptr(out),
                                             self._np_ptr(idx), self._np_ptr(w))
        self._check(rc, "neon_moe_forward_host")
        return (out, idx, w) if want_routing else out

    def run_host_ptr(self, hidden_ptr: int, T: int, logit_bias_ptr: int | None, out_ptr: int) -> None:
        """Host pass on raw (e.g. pinned) addresses, no Python-side copies."""
        self._check(self._lib.neon_moe_forward_host(self._h, hidden_ptr, T, logit_bias_ptr, out_ptr, None, None),
                    "neon_moe_forward_host")

    def run_host_batches(self, hidden_ptrs, T: int, logit_bias_ptr, out_ptrs) -> None:
        """A run of passes over host buffers given by address (pinned memory for real overlap):
        uploads, layer passes and downloads of consecutive batches are pipelined."""
        n = len(hidden_ptrs)
        assert len(out_ptrs) == n
        hp = (ctypes.c_void_p * n)(*hidden_ptrs)
        op = (ctypes.c_void_p * n)(*out_ptrs)
        self._check(self._lib.neon_moe_forward_host_batches(self._h, hp, n, int(T),
                                                            None if not logit_bias_ptr else ctypes.c_void_p(logit_bias_ptr), op),
                    "neon_moe_forward_host_batches")

    def read_dispatch(self):
        n = ctypes.c_int(0)
        self._check(self._lib.neon_moe_read_dispatch(self._h, None, None, None, None, ctypes.byref(n)), "read_dispatch")
        el = self.shape.n_experts // self.ep_size
        count = np.zeros(el, np.int32)
        offset = np.zeros(el + 1, np.int32)
        perm = np.zeros(n.value, np.int32)
        inv = np.zeros(n.value, np.int32)
        self._check(self._lib.neon_moe_read_dispatch(self._h, self._np_ptr(count), self._np_ptr(offset),
                                                     self._np_ptr(perm), self._np_ptr(inv), ctypes.byref(n)),
                    "read_dispatch")
        return count, offset, perm, inv

    def set_option(self, name: str, value: int) -> None:
        self._check(self._lib.neon_moe_set_option(self._h, name.encode(), int(value)), "neon_moe_set_option")

    def profile(self, enable: bool) -> None:
        self._check(self._lib.neon_moe_profile(self._h, int(enable)), "neon_moe_profile")

    def read_profile(self):
        """Summed stage times in ms since the last read: dict + number of forwards."""
        ms = (ctypes.c_double * 4)()
        n = ctypes.c_int(0)
        self._check(self._lib.neon_moe_read_profile(self._h, ms, ctypes.byref(n)), "neon_moe_read_profile")
        return dict(zip(("route_dispatch", "gate_up", "down", "combine"), list(ms))), n.value

    def status(self) -> int:
        word = ctypes.c_int(0)
        self._lib.neon_moe_status(self._h, ctypes.byref(word))
        return word.value

    @property
    def launch_count(self) -> int:
        return int(self._lib.neon_moe_launch_count(self._h))

    def pair_ctas(self) -> int:
        """CTAs the paired (two-SM MMA) grouped GEMM was last launched with; 0 if it has not run."""
        return int(self._lib.neon_moe_pair_ctas(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.neon_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ep_plan(all_counts: np.ndarray, rank: int, cap: int | None = None):
    """Host-side exchange plan (``neon_moe_ep_plan``): ``all_counts[ep_size, n_experts]`` ->
    (send_rows, send_off, recv_rows, recv_off, row_expert).  Needs no GPU."""
    lib = _lib.load()
    all_counts = np.ascontiguousarray(all_counts, np.int32)
    G, E = all_counts.shape
    cap = int(all_counts.sum()) if cap is None else cap
    outs = [np.zeros(G, np.int32) for _ in range(4)]
    row_expert = np.zeros(max(cap, 1), np.int32)
    n_recv = ctypes.c_int(0)
    rc = lib.neon_moe_ep_plan(ctypes.c_void_p(all_counts.ctypes.data), G, E, rank,
                              *[ctypes.c_void_p(o.ctypes.data) for o in outs],
                              ctypes.c_void_p(row_expert.ctypes.data), cap, ctypes.byref(n_recv))
    if rc != 0:
        raise RuntimeError(f"neon_moe_ep_plan failed ({rc})")
    return (*outs, row_expert[:n_recv.value])
