"""ctypes binding of ``libneon_moe.so`` (the C ABI in ``include/neon_moe.h``).

The library is the only compute path: if it is missing or fails to load, importing
callers get an ImportError; nothing falls back to the CPU.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "libneon_moe.so")

c_int = ctypes.c_int
c_void_p = ctypes.c_void_p
c_float_p = ctypes.c_void_p  # raw addresses; device or host depending on the entry point


class NeonMoeConfig(ctypes.Structure):
    """Mirror of ``neon_moe_config``."""
    _fields_ = [("hidden", c_int), ("inter", c_int), ("n_experts", c_int), ("top_k", c_int),
                ("swiglu_limit", ctypes.c_float), ("swiglu_alpha", ctypes.c_float),
                ("max_tokens", c_int), ("ep_rank", c_int), ("ep_size", c_int), ("device", c_int)]


class NeonDecoderConfig(ctypes.Structure):
    """Mirror of ``neon_decoder_config`` (include/neon_decoder.h)."""
    _fields_ = [("n_layers", c_int), ("hidden", c_int), ("n_q_heads", c_int), ("n_kv_heads", c_int),
                ("head_dim", c_int), ("vocab", c_int), ("max_batch", c_int), ("max_ctx", c_int), ("window", c_int),
                ("rope_theta", ctypes.c_float), ("rope_factor", ctypes.c_float), ("rope_orig_ctx", ctypes.c_float),
                ("rope_beta_fast", ctypes.c_float), ("rope_beta_slow", ctypes.c_float), ("rms_eps", ctypes.c_float),
                ("inter", c_int), ("n_experts", c_int), ("top_k", c_int),
                ("swiglu_limit", ctypes.c_float), ("swiglu_alpha", ctypes.c_float), ("device", c_int)]


class NeonWaterConfig(ctypes.Structure):
    """Mirror of ``neon_water_config`` (include/neon_water.h)."""
    _fields_ = [("n_particles", c_int), ("nx", c_int), ("ny", c_int), ("nz", c_int),
                ("cell_size", ctypes.c_float), ("over_relaxation", ctypes.c_float), ("rest_density", ctypes.c_float),
                ("damping", ctypes.c_float), ("mass", ctypes.c_float), ("dt", ctypes.c_float),
                ("box_min", ctypes.c_float * 3), ("box_max", ctypes.c_float * 3), ("gravity", ctypes.c_float * 3),
                ("collision_substeps", c_int), ("jacobi_iterations", c_int), ("device", c_int)]


class NeonSvgfConfig(ctypes.Structure):
    """Mirror of ``neon_svgf_config`` (include/neon_svgf.h)."""
    _fields_ = [("width", c_int), ("height", c_int), ("atrous_iterations", c_int), ("device", c_int)]


class NeonPtConfig(ctypes.Structure):
    """Mirror of ``neon_pt_config`` (include/neon_pt.h)."""
    _fields_ = [("width", c_int), ("height", c_int), ("n_lights", c_int), ("device", c_int)]


# name -> (restype, argtypes); must list every symbol include/neon_pt.h declares
PT_SIGNATURES = {
    "neon_pt_create": (c_int, [ctypes.POINTER(NeonPtConfig), c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "neon_pt_render": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_float, c_void_p, c_void_p]),
    "neon_pt_render_host": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_float, c_void_p]),
    "neon_pt_rays": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint64)]),
    "neon_pt_bvh_info": (c_int, [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "neon_pt_status": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "neon_pt_launch_count": (ctypes.c_int64, [c_void_p]),
    "neon_pt_last_error": (ctypes.c_char_p, [c_void_p]),
    "neon_pt_destroy": (c_int, [c_void_p]),
}

# name -> (restype, argtypes); must list every symbol include/neon_water.h declares
WATER_SIGNATURES = {
    "neon_water_create": (c_int, [ctypes.POINTER(NeonWaterConfig), c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "neon_water_destroy": (c_int, [c_void_p]),
    "neon_water_last_error": (ctypes.c_char_p, [c_void_p]),
    "neon_water_set_particles": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "neon_water_step": (c_int, [c_void_p, c_int, c_void_p]),
    "neon_water_step_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "neon_water_particles_device": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p)]),
    "neon_water_read_particles": (c_int, [c_void_p, c_void_p, c_void_p]),
    "neon_water_read_grid": (c_int, [c_void_p, ctypes.c_char_p, c_void_p, ctypes.c_uint64]),
    "neon_water_status": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "neon_water_profile_step": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_double), c_void_p]),
    "neon_water_set_option": (c_int, [c_void_p, ctypes.c_char_p, ctypes.c_int64]),
    "neon_water_launch_count": (ctypes.c_int64, [c_void_p]),
}

# name -> (restype, argtypes); must list every symbol include/neon_svgf.h declares
SVGF_SIGNATURES = {
    "neon_svgf_create": (c_int, [ctypes.POINTER(NeonSvgfConfig), ctypes.POINTER(c_void_p)]),
    "neon_svgf_destroy": (c_int, [c_void_p]),
    "neon_svgf_last_error": (ctypes.c_char_p, [c_void_p]),
    "neon_svgf_set_history": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "neon_svgf_denoise": (c_int, [c_void_p] + [c_void_p] * 5 + [c_void_p]),
    "neon_svgf_denoise_host": (c_int, [c_void_p] + [c_void_p] * 5 + [c_void_p]),
    "neon_svgf_read": (c_int, [c_void_p, ctypes.c_char_p, c_void_p, ctypes.c_uint64]),
    "neon_svgf_profile_frame": (c_int, [c_void_p] + [c_void_p] * 5 + [ctypes.POINTER(ctypes.c_double), c_void_p]),
    "neon_svgf_set_option": (c_int, [c_void_p, ctypes.c_char_p, ctypes.c_int64]),
    "neon_svgf_launch_count": (ctypes.c_int64, [c_void_p]),
}

# name -> (restype, argtypes); must list every symbol include/neon_decoder.h declares
DECODER_SIGNATURES = {
    "neon_decoder_create": (c_int, [ctypes.POINTER(NeonDecoderConfig), ctypes.POINTER(c_void_p)]),
    "neon_decoder_destroy": (c_int, [c_void_p]),
    "neon_decoder_last_error": (ctypes.c_char_p, [c_void_p]),
    "neon_decoder_set_embeddings": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "neon_decoder_set_attention": (c_int, [c_void_p, c_int] + [c_void_p] * 7 + [c_int]),
    "neon_decoder_set_moe": (c_int, [c_void_p, c_int] + [c_void_p] * 8 + [c_int]),
    "neon_decoder_load_kv": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int]),
    "neon_decoder_step": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "neon_decoder_step_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "neon_decoder_read": (c_int, [c_void_p, ctypes.c_char_p, c_void_p, ctypes.c_uint64]),
    "neon_decoder_set_option": (c_int, [c_void_p, ctypes.c_char_p, ctypes.c_int64]),
    "neon_decoder_launch_count": (ctypes.c_int64, [c_void_p]),
    "neon_decoder_step_bytes": (c_int, [c_void_p, c_void_p, c_int, ctypes.POINTER(ctypes.c_double)]),
}

# name -> (restype, argtypes); must list every symbol include/neon_moe.h declares
SIGNATURES = {
    "neon_moe_create": (c_int, [ctypes.POINTER(NeonMoeConfig), ctypes.POINTER(c_void_p)]),
    "neon_moe_set_weights": (c_int, [c_void_p] * 9 + [c_int]),
    "neon_moe_save_weights": (c_int, [c_void_p, ctypes.c_char_p]),
    "neon_moe_load_weights_file": (c_int, [c_void_p, ctypes.c_char_p]),
    "neon_moe_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "neon_moe_forward_static": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "neon_moe_ep_unique_id": (c_int, [c_void_p]),
    "neon_moe_ep_init": (c_int, [c_void_p, c_void_p]),
    "neon_moe_forward_ep": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "neon_moe_ep_times": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(c_int)]),
    "neon_moe_ep_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 ctypes.POINTER(c_int)]),
    "neon_moe_ep_subpasses": (c_int, [c_void_p]),
    "neon_moe_ep_peer_export": (c_int, [c_void_p, c_void_p]),
    "neon_moe_ep_peer_import": (c_int, [c_void_p, c_void_p]),
    "neon_moe_ep_overflow": (c_int, [c_void_p, c_int, c_int, c_void_p, ctypes.POINTER(c_int)]),
    "neon_moe_forward_host": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "neon_moe_forward_host_batches": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "neon_moe_read_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_int)]),
    "neon_moe_status": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "neon_moe_set_option": (c_int, [c_void_p, ctypes.c_char_p, ctypes.c_int64]),
    "neon_moe_profile": (c_int, [c_void_p, c_int]),
    "neon_moe_read_profile": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(c_int)]),
    "neon_moe_pair_ctas": (c_int, [c_void_p]),
    "neon_moe_tma_rate": (c_int, [c_int, c_int, c_int, ctypes.c_int64, c_int, ctypes.POINTER(ctypes.c_double),
                                  ctypes.POINTER(ctypes.c_int64)]),
    "neon_moe_launch_count": (ctypes.c_int64, [c_void_p]),
    "neon_moe_last_error": (ctypes.c_char_p, [c_void_p]),
    "neon_moe_destroy": (c_int, [c_void_p]),
    "neon_moe_version": (ctypes.c_char_p, []),
    "neon_moe_mma_pair_probe": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, ctypes.POINTER(ctypes.c_int64)]),
    "neon_moe_mma_rate": (c_int, [c_int, c_int, c_int, c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int64)]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library and bind every entry point; raises ImportError when the
    CUDA extension has not been built (``python -m neonengine_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise ImportError(f"{SO_PATH} is missing: build it with `python -m neonengine_b200.build` "
                          "(there is no CPU fallback)")
    lib = ctypes.CDLL(SO_PATH)
    for name, (res, args) in {**SIGNATURES, **DECODER_SIGNATURES, **WATER_SIGNATURES, **SVGF_SIGNATURES, **PT_SIGNATURES}.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
