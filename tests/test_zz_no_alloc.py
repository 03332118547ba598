"""The allocation-free entry point, ``neon_moe_forward_static``.

Some users of the library cannot allocate device memory at the point where they need a
layer pass: a plugin confined to its host application's memory budget, a decode loop
that must not hit the CUDA allocator's lock and implicit synchronisation, or a thread
that needs a pass while the handle's own workspaces are in use on another stream.  For
them the library keeps the pass's intermediates in a 2 MiB array built into its image.

This file is collected last on purpose, so a run that stops at the first failure has
already run every other test.  The check: through the C ABI, two passes in a row (the
second one smaller, so stale contents of the shared array would show) must reproduce
the regular entry point's outputs within the tolerance the other parity tests use, and
a batch too large for the array must be refused with a clear message.
"""
import numpy as np
import pytest

from helpers import assert_close
from neonengine_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_regular_forward_twice():
    import torch
    from neonengine_b200.moe_layer_system import MoeLayerSystem
    assert torch.cuda.is_available()
    shape = synth.MoeShape(hidden=2880, inter=2880, n_experts=8, top_k=4)
    W = synth.make_weights(shape, 21)
    lb = synth.zipf_logit_bias(shape.n_experts)
    layer = MoeLayerSystem(shape, W, max_tokens=32, device=0)
    d_lb = torch.from_numpy(lb).cuda()
    for call, (T, bias) in enumerate([(20, d_lb), (3, None)]):
        hidden = synth.make_hidden(T, W, 21, logit_bias=lb if bias is not None else None, stream=call)
        h = torch.from_numpy(hidden.view(np.int16)).cuda()
        ref, ridx, rw = layer.run(h, logit_bias=bias, want_routing=True)
        out = torch.empty_like(ref)                 # caller-owned output, made before the call
        got, idx, w = layer.run_static(h, logit_bias=bias, out=out, want_routing=True)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(idx.cpu().numpy(), ridx.cpu().numpy())
        np.testing.assert_allclose(w.cpu().numpy(), rw.cpu().numpy(), rtol=0, atol=2e-6)
        assert_close(got.cpu().numpy(), ref.cpu().numpy(), f"static call {call}")
    # beyond the built-in array: refused, nothing launched
    big = torch.zeros((23, shape.hidden), dtype=torch.int16, device="cuda")
    with pytest.raises(RuntimeError, match="built-in array holds"):
        layer.run_static(big)
    layer.close()
