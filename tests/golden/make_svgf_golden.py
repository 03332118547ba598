"""Generates tests/golden/svgf_small.npz from the reference engine's own denoiser shaders compiled
for the CPU (oracle/svgf_ref_build.py -> oracle/_ref/libsvgf_ref.so; needs the reference
checkout).  Small case so the fixture stays a few tens of KB: 48 x 32 pixels, 3 frames of the
seeded synthetic scene (neonengine_b200/svgf_synth.py), the reference's 3 filter iterations,
the bodies of the shaders live (their leading `return;` not honoured).  Stored: the outputs only
(denoised image per frame, the final state); the inputs are regenerated from the seed.

    python tests/golden/make_svgf_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from neonengine_b200 import svgf_synth  # noqa: E402
from oracle import svgf, svgf_ref_build  # noqa: E402

W, H, FRAMES, ITERATIONS = 48, 32, 3, 3

if __name__ == "__main__":
    if svgf_ref_build.build(force=True) is None:
        raise SystemExit("the reference checkout is not available: cannot regenerate the fixture")
    st = svgf.State.zeros(W, H)
    out = {}
    for i in range(FRAMES):
        g, image = svgf_synth.make_frame(W, H, i)
        if i == 0:
            out["input0_crc"] = np.array([int(np.frombuffer(b"".join(a.tobytes() for a in g) + image.tobytes(), np.uint8).sum())])
        svgf.ref_frame(g, image, st, ITERATIONS)
        out[f"image{i}"] = image.copy()
    out.update(colour_a=st.colour_a, colour_b=st.colour_b, moments=st.data, ping_pong=np.array([st.ping_pong]))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "svgf_small.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")
