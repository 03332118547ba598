"""CPU tests of the C-ABI library: it loads, exports every declared symbol, and refuses
to compute without a GPU (no CPU fallback)."""
import ctypes
import os
import re

import pytest

from neonengine_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_symbols(header="neon_moe.h", prefix="neon_moe_"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z_0-9]+)\s*\(", text)))


def test_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in neon_moe.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "python binding table out of sync with the header"


def test_exports_every_declared_decoder_symbol(lib):
    names = declared_symbols("neon_decoder.h", "neon_decoder_")
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in neon_decoder.h but not exported"
    assert set(names) == set(_lib.DECODER_SIGNATURES), "python binding table out of sync with the header"


def test_exports_every_declared_water_symbol(lib):
    names = declared_symbols("neon_water.h", "neon_water_")
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in neon_water.h but not exported"
    assert set(names) == set(_lib.WATER_SIGNATURES), "python binding table out of sync with the header"


def test_exports_every_declared_svgf_symbol(lib):
    names = declared_symbols("neon_svgf.h", "neon_svgf_")
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in neon_svgf.h but not exported"
    assert set(names) == set(_lib.SVGF_SIGNATURES), "python binding table out of sync with the header"


def test_exports_every_declared_path_tracer_symbol(lib):
    names = declared_symbols("neon_pt.h", "neon_pt_")
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in neon_pt.h but not exported"
    assert set(names) == set(_lib.PT_SIGNATURES), "python binding table out of sync with the header"


def test_water_create_rejects_bad_config(lib):
    h = ctypes.c_void_p()
    cfg = _lib.NeonWaterConfig(8, 1, 4, 4, 0.1, 1.0, 1.0, 0.0, 1.0, 0.002)  # one cell along x
    buf = (ctypes.c_float * 32)()
    assert lib.neon_water_create(ctypes.byref(cfg), buf, 0, ctypes.byref(h)) == 1
    assert b"grid" in lib.neon_water_last_error(None)
    assert lib.neon_water_step(None, 1, None) == 1


def test_decoder_create_rejects_bad_config(lib):
    h = ctypes.c_void_p()
    cfg = _lib.NeonDecoderConfig(1, 128, 8, 2, 32, 1000, 2, 64, 0, 150000.0, 32.0, 4096.0, 32.0, 1.0, 1e-5,
                                 64, 8, 4, 7.0, 1.702, 0)  # head_dim 32 is not supported
    assert lib.neon_decoder_create(ctypes.byref(cfg), ctypes.byref(h)) == 1
    assert b"head_dim" in lib.neon_decoder_last_error(None)
    assert lib.neon_decoder_step(None, None, None, 1, None, None, None) == 1


def test_version(lib):
    assert b"sm_100a" in lib.neon_moe_version()


def test_create_rejects_bad_config(lib):
    h = ctypes.c_void_p()
    cfg = _lib.NeonMoeConfig(100, 64, 8, 4, 7.0, 1.702, 4, 0, 1, 0)  # hidden not a multiple of 64
    assert lib.neon_moe_create(ctypes.byref(cfg), ctypes.byref(h)) == 1
    assert b"multiples of 64" in lib.neon_moe_last_error(None)
    cfg = _lib.NeonMoeConfig(64, 64, 8, 9, 7.0, 1.702, 4, 0, 1, 0)   # top_k too large
    assert lib.neon_moe_create(ctypes.byref(cfg), ctypes.byref(h)) == 1
    cfg = _lib.NeonMoeConfig(64, 64, 8, 4, 7.0, 1.702, 4, 3, 2, 0)   # rank >= size
    assert lib.neon_moe_create(ctypes.byref(cfg), ctypes.byref(h)) == 1


def test_no_cpu_fallback(lib):
    """Without a GPU a valid create must fail with the CUDA error code, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    h = ctypes.c_void_p()
    cfg = _lib.NeonMoeConfig(64, 64, 8, 4, 7.0, 1.702, 4, 0, 1, 0)
    assert lib.neon_moe_create(ctypes.byref(cfg), ctypes.byref(h)) == 2
    assert not h.value


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "neonengine_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"(import\s+oracle|from\s+oracle|moe_oracle|oracle/)", text), \
                    f"{f} reaches into the oracle"


def test_cpp_wrappers_compile():
    """The header-only engine-style C++ owners of the handles compile as C++17."""
    import subprocess
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "check.cpp")
        with open(src, "w") as f:
            f.write('#include "lve_moe_layer_system.hpp"\n#include "lve_water_physics.hpp"\n#include "lve_svgf_denoiser.hpp"\nint main() { return 0; }\n')
        res = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I" + os.path.join(ROOT, "include"), src],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
