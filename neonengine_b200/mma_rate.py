"""Host side of ``neon_moe_mma_rate`` (include/neon_moe.h): the measured ceiling of the block-scaled
tensor-core instructions the grouped GEMM issues, operands resident in shared memory."""
from __future__ import annotations

import ctypes

from . import _lib

KINDS = {"mxf8f6f4": 0, "mxf4": 1}


def measure(kind: str = "mxf8f6f4", n: int = 128, chunks: int = 8192, device: int = 0, n_sms: int | None = None) -> dict:
    """Returns {"tflops": whole-GPU rate from the launch duration, "cycles_per_mma": on one SM,
    "flops_per_cycle_per_sm", "ms"} for 128 x n instructions of the given kind."""
    lib = _lib.load()
    ms, cycles = ctypes.c_double(), ctypes.c_int64()
    rc = lib.neon_moe_mma_rate(device, KINDS[kind], n, chunks, ctypes.byref(ms), ctypes.byref(cycles))
    if rc != 0:
        raise RuntimeError(f"neon_moe_mma_rate failed ({rc})")
    if n_sms is None:
        import torch
        n_sms = torch.cuda.get_device_properties(device).multi_processor_count
    per_group = 2.0 * 128 * n * 128            # one group covers K = 128
    mmas = chunks * (4 if kind == "mxf8f6f4" else 2)
    return {"kind": kind, "n": n, "chunks": chunks, "ms": ms.value,
            "tflops": per_group * chunks * n_sms / (ms.value * 1e-3) / 1e12,
            "cycles_per_mma": cycles.value / mmas,
            "flops_per_cycle_per_sm": per_group * chunks / cycles.value}
