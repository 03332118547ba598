"""The allocation-free entry point, ``neon_moe_forward_static``.

Some users of the library cannot allocate device memory at the point where they need a
layer pass: a plugin confined to its host application's memory budget, a decode loop
that must not hit the CUDA allocator's lock and implicit synchronisation, or a thread
that needs a pass while the handle's own workspaces are in use on another stream.  For
them the library keeps the pass's intermediates in a 2 MiB array built into its image.
Whoever sets the layer up (and may allocate) asks once for the weight layout this entry
point reads (option ``mma16_layout``); the passes themselves then allocate nothing.

This file is collected last on purpose, so a run that stops at the first failure has
already run every other test.  The checks, all through the C ABI: two passes in a row
(the second one smaller, so stale contents of the shared array would show) must match
the CPU oracle (routing bit-exact, outputs within the contract tolerance) and the regular
entry point; the device's free memory must be the same after the passes as before them;
the caller's current device must be untouched; a batch too large for the array and a
handle without the layout must be refused with clear messages.
"""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import assert_close
from neonengine_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_oracle_and_regular_forward_twice():
    import torch
    from neonengine_b200.moe_layer_system import MoeLayerSystem
    assert torch.cuda.is_available()
    shape = synth.MoeShape(hidden=2880, inter=2880, n_experts=8, top_k=4)
    W = synth.make_weights(shape, 21)
    lb = synth.zipf_logit_bias(shape.n_experts)
    layer = MoeLayerSystem(shape, W, max_tokens=32, device=0)
    lib = layer._lib
    probe = torch.zeros((1, shape.hidden), dtype=torch.int16, device="cuda")
    with pytest.raises(RuntimeError, match="mma16_layout"):
        layer.run_static(probe)                         # the layout has not been asked for yet
    layer.set_option("mma16_layout", 1)                 # set-up time: this call allocates
    d_lb = torch.from_numpy(lb).cuda()
    cases = []
    for call, (T, bias) in enumerate([(20, d_lb), (3, None)]):
        hidden = synth.make_hidden(T, W, 21, logit_bias=lb if bias is not None else None, stream=call)
        h = torch.from_numpy(hidden.view(np.int16)).cuda()
        ref, ridx, rw = layer.run(h, logit_bias=bias, want_routing=True)
        # everything the pass writes is made before it, so the pass itself has nothing to allocate
        out = torch.empty_like(ref)
        idx = torch.empty_like(ridx)
        w = torch.empty_like(rw)
        cases.append((hidden, bias, h, ref, ridx, rw, out, idx, w))
    layer.run_static(cases[0][2], logit_bias=cases[0][1], out=torch.empty_like(cases[0][3]))   # first call: symbol look-up
    torch.cuda.synchronize()
    st = torch.cuda.current_stream().cuda_stream
    free_before = torch.cuda.mem_get_info()[0]
    for hidden, bias, h, ref, ridx, rw, out, idx, w in cases:
        rc = lib.neon_moe_forward_static(layer._h, h.data_ptr(), h.shape[0], None if bias is None else bias.data_ptr(),
                                         out.data_ptr(), idx.data_ptr(), w.data_ptr(), st)
        assert rc == 0, lib.neon_moe_last_error(None).decode()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free pass changed the device's free memory"
    assert torch.cuda.current_device() == 0
    for call, (hidden, bias, h, ref, ridx, rw, out, idx, w) in enumerate(cases):
        want, oidx, ow = oracle.moe_forward(hidden, W, logit_bias=lb if bias is not None else None)
        np.testing.assert_array_equal(idx.cpu().numpy(), oidx)
        np.testing.assert_allclose(w.cpu().numpy(), ow, rtol=0, atol=2e-6)
        assert_close(out.cpu().numpy(), want, f"static call {call} vs oracle")
        np.testing.assert_array_equal(idx.cpu().numpy(), ridx.cpu().numpy())
        assert_close(out.cpu().numpy(), ref.cpu().numpy(), f"static call {call} vs regular entry point")
    # beyond the built-in array: refused, nothing launched
    big = torch.zeros((23, shape.hidden), dtype=torch.int16, device="cuda")
    with pytest.raises(RuntimeError, match="built-in array holds"):
        layer.run_static(big)
    layer.close()
