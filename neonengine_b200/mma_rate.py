"""Host side of ``neon_moe_mma_rate`` (include/neon_moe.h): the measured ceiling of the block-scaled
tensor-core instructions the grouped GEMM issues, operands resident in shared memory."""
from __future__ import annotations

import ctypes

from . import _lib

KINDS = {"mxf8f6f4": 0, "mxf4": 1, "mxf8f6f4+sf": 2, "mxf4+sf": 3}   # "+sf": one scale-atom copy per K = 128 group


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
    mmas = chunks * (4 if kind.startswith("mxf8f6f4") else 2)
    return {"kind": kind, "n": n, "chunks": chunks, "ms": ms.value,
            "tflops": per_group * chunks * n_sms / (ms.value * 1e-3) / 1e12,
            "cycles_per_mma": cycles.value / mmas,
            "flops_per_cycle_per_sm": per_group * chunks / cycles.value}


def tma_copy_rate(packed: bool = False, stages: int = 4, buffer_mib: int = 8, loads: int = 2048, device: int = 0,
                  n_sms: int | None = None) -> dict:
    """Host side of ``neon_moe_tma_rate``: {"gbs_per_sm": bytes of global memory one SM's TMA unit brought in per
    second (by its own clock count at the SM clock of the launch), "gbs": whole GPU from the launch duration,
    "cycles_per_load": SM clocks per 16 KB box pair}."""
    lib = _lib.load()
    ms, cycles = ctypes.c_double(), ctypes.c_int64()
    rc = lib.neon_moe_tma_rate(device, int(packed), stages, buffer_mib << 20, loads, ctypes.byref(ms), ctypes.byref(cycles))
    if rc != 0:
        raise RuntimeError(f"neon_moe_tma_rate failed ({rc})")
    if n_sms is None:
        import torch
        n_sms = torch.cuda.get_device_properties(device).multi_processor_count
    return {"packed": packed, "stages": stages, "buffer_mib": buffer_mib, "ms": ms.value,
            "gbs": loads * 16384.0 * n_sms / (ms.value * 1e-3) / 1e9,
            "cycles_per_load": cycles.value / loads, "bytes_per_cycle_per_sm": loads * 16384.0 / cycles.value}
