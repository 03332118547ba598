"""In-tree build of ``libneon_moe.so`` (sm_100a only) with nvcc.

``python -m neonengine_b200.build`` compiles the CUDA sources under ``csrc/`` into
``neonengine_b200/libneon_moe.so``.  nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(HERE, "libneon_moe.so")
APP = os.path.join(HERE, "moe_app")
SOURCES = ["neon_moe.cu", "neon_decoder.cu", "neon_water.cu", "neon_svgf.cu", "neon_pt.cu"]
# the water step reproduces the reference shader's float arithmetic bit for bit: no fused multiply-add there
SOURCE_FLAGS = {"neon_water.cu": ["-fmad=false"], "neon_svgf.cu": ["-fmad=false"], "neon_pt.cu": ["-fmad=false"]}
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-cudart", "static"]
if os.environ.get("NEON_MOE_INSTRUMENT"):   # measurement aids (clock stamps, debug options); never in the shipped library
    NVCC_FLAGS.append("-DNEON_MOE_INSTRUMENT")


def _newest_source() -> float:
    newest = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in os.listdir(root):
            newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every source to an object (in parallel) and links the shared library."""
    if not force and os.path.exists(SO) and os.path.getmtime(SO) >= _newest_source():
        return SO
    objdir = os.path.join(HERE, "_obj")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = ["nvcc", *NVCC_FLAGS, *SOURCE_FLAGS.get(src, []), *(["-Xptxas", "-v"] if verbose else []), "-c",
               os.path.join(CSRC, src), "-o", obj]
        procs.append((cmd, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for cmd, obj, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out)
        if proc.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        objs.append(obj)
    cmd = ["nvcc", *NVCC_FLAGS, "-shared", *objs, "-o", SO, "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc link failed: " + " ".join(cmd))
    # the headless application loop (engine-style owner of the layer), linked against the library
    cmd = ["nvcc", "-O2", "-std=c++17", "-cudart", "static", os.path.join(CSRC, "moe_app.cpp"), "-o", APP,
           "-L" + HERE, "-lneon_moe", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("building moe_app failed: " + " ".join(cmd))
    return SO


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
