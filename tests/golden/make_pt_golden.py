"""Writes tests/golden/pt_small.npz: frames of the path tracer's small test scenes rendered by the
reference engine's OWN shaders compiled for the CPU (oracle/pt_ref_build.py -> oracle/_ref/libpt_ref.so).
Run where the reference checkout is present:  python tests/golden/make_pt_golden.py
The fixture keeps the pin on machines without the checkout: the restatement and the CUDA kernel must
reproduce these bytes."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from neonengine_b200 import pt_synth  # noqa: E402
from oracle import pt  # noqa: E402

CASES = [("small_seed1", 1, 96, 64, 3.0), ("small_seed4", 4, 80, 48, 11.5)]


def main():
    out = {}
    for name, seed, w, h, frame_id in CASES:
        sc = pt_synth.small_scene(seed)
        ip, iv = pt_synth.camera(w, h)
        img, rays = pt.ref_render(sc, ip, iv, frame_id, w, h)
        out[name + "_image"] = img
        out[name + "_rays"] = np.int64(rays)
        out[name + "_params"] = np.array([seed, w, h, frame_id], np.float64)
    # a crop of the engine's own configuration: Cornell box, 800 x 600 camera, rows 300..307
    sc = pt_synth.cornell_box(0)
    ip, iv = pt_synth.camera(800, 600)
    img, rays = pt.ref_render(sc, ip, iv, 5.0, 800, 600)
    out["cornell_rows_300_308"] = img[300:308].copy()
    out["cornell_rays"] = np.int64(rays)
    out["cornell_checksum"] = np.int64(int(img.astype(np.int64).sum()))
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "pt_small.npz"), **out)
    print({k: (v.shape if hasattr(v, "shape") and v.shape else v) for k, v in out.items()})


if __name__ == "__main__":
    main()
