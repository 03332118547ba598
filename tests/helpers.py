"""Shared helpers for the parity tests."""
import os

import numpy as np

from neonengine_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MAX_ABS_TOL = 2e-2      # contract: max-abs error versus the fp32-accumulated (here fp64) result
MEAN_REL_TOL = 5e-3     # contract: mean|y - ref| / mean|ref|


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    k = int(z["top_k"])
    E, H = z["router_w"].shape
    I = z["down_blocks"].shape[2] * 2
    shape = synth.MoeShape(hidden=H, inter=I, n_experts=E, top_k=k)
    W = synth.MoeWeights(shape, z["router_w"], z["router_b"], z["gate_up_blocks"], z["gate_up_scales"],
                         z["gate_up_bias"], z["down_blocks"], z["down_scales"], z["down_bias"])
    lb = z["logit_bias"] if z["logit_bias"].size else None
    return shape, W, z["hidden"], lb, z


def errors(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    max_abs = float(np.abs(got - ref).max()) if ref.size else 0.0
    mean_rel = float(np.abs(got - ref).mean() / max(np.abs(ref).mean(), 1e-30)) if ref.size else 0.0
    return max_abs, mean_rel


def assert_close(got, ref, what=""):
    max_abs, mean_rel = errors(got, ref)
    assert max_abs <= MAX_ABS_TOL and mean_rel <= MEAN_REL_TOL, \
        f"{what}: max_abs={max_abs:.3e} (tol {MAX_ABS_TOL}), mean_rel={mean_rel:.3e} (tol {MEAN_REL_TOL})"
    return max_abs, mean_rel
