"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Routing and dispatch are integer work and must be bit-exact;
outputs must meet the contract tolerance (max-abs <= 2e-2 and mean-rel <= 5e-3)."""
import numpy as np
import pytest

import oracle
from helpers import assert_close, load_golden
from neonengine_b200 import synth

pytestmark = pytest.mark.gpu


def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


def make_layer(shape, W, max_tokens):
    from neonengine_b200.moe_layer_system import MoeLayerSystem
    return MoeLayerSystem(shape, W, max_tokens=max_tokens, device=0)


def run_device(layer, hidden, logit_bias=None):
    torch = torch_cuda()
    h = torch.from_numpy(hidden.view(np.int16)).cuda()
    lb = None if logit_bias is None else torch.from_numpy(np.asarray(logit_bias, np.float32)).cuda()
    out, idx, w = layer.run(h, logit_bias=lb, want_routing=True)
    torch.cuda.synchronize()
    return out.cpu().numpy(), idx.cpu().numpy(), w.cpu().numpy()


def check_against_oracle(layer, W, hidden, logit_bias=None, tokens=None, what=""):
    out, idx, w = run_device(layer, hidden, logit_bias)
    ridx, rw = oracle.route(hidden, W.router_w, W.router_b, W.shape.top_k, logit_bias)
    np.testing.assert_array_equal(idx, ridx, err_msg=f"{what}: routing indices differ")
    np.testing.assert_allclose(w, rw, rtol=0, atol=2e-6, err_msg=f"{what}: routing weights")
    ref = oracle.experts(hidden, ridx, rw, W, tokens=tokens)
    got = out if tokens is None else out[tokens]
    err = assert_close(got, ref, what)
    # dispatch arrays: bit-exact with the oracle's stable counting sort
    count, offset, perm, inv = layer.read_dispatch()
    rc, ro, rp, ri = oracle.dispatch(ridx, W.shape.n_experts)
    np.testing.assert_array_equal(count, rc)
    np.testing.assert_array_equal(offset, ro)
    np.testing.assert_array_equal(perm, rp)
    np.testing.assert_array_equal(inv, ri)
    assert layer.status() == 0
    return out, err


@pytest.mark.parametrize("name", ["small_seeded", "small_seeded_zipf", "integer_kat", "clamp_negative", "all_ties"])
def test_golden_vectors(name):
    shape, W, hidden, lb, z = load_golden(name)
    layer = make_layer(shape, W, max_tokens=16)
    out, idx, w = run_device(layer, hidden, lb)
    np.testing.assert_array_equal(idx, z["idx"])
    np.testing.assert_allclose(w, z["w"], rtol=0, atol=2e-6)
    ref = z["out"]
    if name == "integer_kat" or name == "all_ties":   # |out| ~ 3584: compare relatively
        np.testing.assert_allclose(out, ref, rtol=2e-6)
    else:
        assert_close(out, ref, name)
    # the host-buffer entry point gives the same bits
    out_h, idx_h, w_h = layer.run_host(hidden, lb, want_routing=True)
    np.testing.assert_array_equal(out_h, out)
    np.testing.assert_array_equal(idx_h, idx)
    layer.close()


@pytest.fixture(scope="module")
def full20b():
    """gpt-oss-20b-shaped layer: H=I=2880, E=32, k=4, benchmark distributions, seed 0."""
    shape = synth.MoeShape()
    W = synth.make_weights(shape, 0)
    layer = make_layer(shape, W, max_tokens=512)
    yield shape, W, layer
    layer.close()


@pytest.fixture(scope="module")
def full20b_prefill():
    """The same layer with room for a 4096-token pass."""
    shape = synth.MoeShape()
    W = synth.make_weights(shape, 0)
    layer = make_layer(shape, W, max_tokens=4096)
    yield shape, W, layer
    layer.close()


def test_config0_decode_single_token(full20b):
    shape, W, layer = full20b
    for stream in range(3):
        hidden = synth.make_hidden(1, W, 0, stream=stream)
        check_against_oracle(layer, W, hidden, what=f"config0 stream {stream}")


@pytest.mark.parametrize("path", [2, 1])
def test_config1_batched_decode_zipf(full20b, path):
    """Both kernel generations: 2 = TMA + tcgen05 block-scaled GEMM (default), 1 = mma.sync."""
    shape, W, layer = full20b
    layer.set_option("path", path)
    try:
        _config1(shape, W, layer)
    finally:
        layer.set_option("path", 2)


def _config1(shape, W, layer):
    lb = synth.zipf_logit_bias(shape.n_experts)
    hidden = synth.make_hidden(64, W, 0, logit_bias=lb)
    out, err = check_against_oracle(layer, W, hidden, logit_bias=lb, what="config1")
    count = layer.read_dispatch()[0]
    assert count.sum() == 256 and count.max() > 3 * count[count > 0].min()  # loads are skewed


@pytest.mark.parametrize("T", [2, 3, 5, 9, 17, 33, 100, 200, 224, 225, 384, 385])
def test_ragged_token_counts(full20b, T):
    """Odd sizes either side of every switch of router kernel and token-tile size (16 / 64 / 224 / 384)."""
    shape, W, layer = full20b
    hidden = synth.make_hidden(T, W, 1, stream=T)
    toks = None if T <= 33 else np.arange(0, T, 7 if T <= 100 else 29, dtype=np.int32)
    check_against_oracle(layer, W, hidden, tokens=toks, what=f"T={T}")


def test_all_tokens_on_the_same_experts(full20b):
    """A large bias on four experts sends every token to them: 28 experts stay empty and
    four experts get all 40 tokens (more than one 8-token MMA tile)."""
    shape, W, layer = full20b
    lb = np.zeros(shape.n_experts, np.float32)
    lb[[3, 7, 20, 31]] = 50.0
    hidden = synth.make_hidden(40, W, 2, logit_bias=lb)
    out, _ = check_against_oracle(layer, W, hidden, logit_bias=lb, what="same experts")
    count = layer.read_dispatch()[0]
    assert sorted(np.nonzero(count)[0].tolist()) == [3, 7, 20, 31] and set(count[count > 0]) == {40}


def test_empty_batch_and_bad_sizes(full20b):
    shape, W, layer = full20b
    out = layer.run_host(np.zeros((0, shape.hidden), np.uint16))
    assert out.shape == (0, shape.hidden)
    with pytest.raises(RuntimeError, match="max_tokens"):
        layer.run_host(np.zeros((513, shape.hidden), np.uint16))


def test_deterministic_and_token_order_invariant(full20b):
    """Two runs give identical bits, and permuting the tokens permutes the output rows
    bit-exactly (each token's reductions do not depend on its position in the batch)."""
    shape, W, layer = full20b
    lb = synth.zipf_logit_bias(shape.n_experts)
    hidden = synth.make_hidden(64, W, 3, logit_bias=lb)
    a = run_device(layer, hidden, lb)[0]
    b = run_device(layer, hidden, lb)[0]
    np.testing.assert_array_equal(a, b)
    perm = np.random.default_rng(0).permutation(64)
    c = run_device(layer, np.ascontiguousarray(hidden[perm]), lb)[0]
    np.testing.assert_array_equal(c, a[perm])


def test_prefill_sized_batch_properties(full20b):
    """T=512 (uniform routing): oracle on a token sample, routing exact for all tokens,
    routing weights sum to one, counts add up."""
    shape, W, layer = full20b
    hidden = synth.make_hidden(512, W, 4)
    toks = np.arange(3, 512, 37, dtype=np.int32)
    out, _ = check_against_oracle(layer, W, hidden, tokens=toks, what="T=512")
    _, idx, w = run_device(layer, hidden)
    np.testing.assert_allclose(w.sum(axis=1), 1.0, atol=1e-6)
    assert layer.read_dispatch()[0].sum() == 512 * 4
    assert np.isfinite(out).all()


def test_large_scales_load_on_the_tensor_core_path():
    """E8M0 bytes up to 140 (scales up to 2^13) are ordinary weights for the tensor-core path:
    outputs stay within the contract's mean relative error and, relative to the largest output,
    within its absolute one.  The mma.sync layout cannot hold them: asking for it fails, and the
    handle keeps working on the tensor-core path."""
    shape, W, hidden, lb, z = load_golden("small_seeded")
    rng = np.random.default_rng(5)
    big = synth.MoeWeights(shape, W.router_w, W.router_b, W.gate_up_blocks, W.gate_up_scales.copy(),
                           W.gate_up_bias, W.down_blocks, W.down_scales.copy(), W.down_bias)
    for sc in (big.gate_up_scales, big.down_scales):
        pick = rng.random(sc.shape) < 0.05
        sc[pick] = rng.integers(129, 141, int(pick.sum()), dtype=np.uint8)
    layer = make_layer(shape, big, 16)
    out, idx, w = run_device(layer, hidden, lb)
    ref, ridx, rw = oracle.moe_forward(hidden, big, logit_bias=lb)
    np.testing.assert_array_equal(idx, ridx)
    scale = np.abs(ref).max()
    assert np.isfinite(out).all() and scale > 1e3
    max_abs = np.abs(out - ref).max() / scale
    mean_rel = np.abs(out - ref).mean() / np.abs(ref).mean()
    assert max_abs <= 1e-5 and mean_rel <= 5e-3, (max_abs, mean_rel)
    with pytest.raises(RuntimeError, match="scale bytes above 128"):
        layer.set_option("path", 1)
    with pytest.raises(RuntimeError, match="scale bytes above 128"):
        layer.set_option("mma16_layout", 1)
    out2, _, _ = run_device(layer, hidden, lb)
    np.testing.assert_array_equal(out2, out)
    layer.close()


def test_mma16_layout_is_built_on_request_only():
    """set_weights keeps one copy of the expert weights; the mma.sync layout appears (and device
    memory shrinks by about the weights' size) only when asked for, and goes away again."""
    torch = torch_cuda()
    shape = synth.MoeShape(hidden=2880, inter=2880, n_experts=8, top_k=4)
    W = synth.make_weights(shape, 3)
    layer = make_layer(shape, W, 8)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    layer.set_option("mma16_layout", 1)
    free1 = torch.cuda.mem_get_info()[0]
    weights = 8 * (2880 * 2880 * 3 // 2)
    assert 0.9 * weights < free0 - free1 < 1.5 * weights
    hidden = synth.make_hidden(5, W, 3)
    a = run_device(layer, hidden)[0]
    layer.set_option("path", 1)
    b = run_device(layer, hidden)[0]
    layer.set_option("path", 2)
    assert_close(b, a, "path 1 vs path 2")
    layer.set_option("mma16_layout", 0)
    assert torch.cuda.mem_get_info()[0] >= free0 - (4 << 20)
    layer.close()


@pytest.mark.parametrize("n_experts", [32, 128])
def test_tensor_core_router_breaks_exact_ties_like_the_others(n_experts):
    """Exact ties and signed zeros through the large-batch routers (T > 384): identical router
    rows give bit-equal logits in every router, so the lower expert id must win; a zero hidden
    state makes every logit the bias alone (+0 and -0 compare equal).  Tensor-core router,
    CUDA-core router and the oracle must agree on every token."""
    torch = torch_cuda()
    shape = synth.MoeShape(hidden=256, inter=64, n_experts=n_experts, top_k=4)
    W = synth.make_weights(shape, 7)
    rw = W.router_w.copy()
    rb = W.router_b.copy()
    rw[5] = rw[2]; rw[9] = rw[2]; rw[n_experts - 1] = rw[0]        # three-way and two-way ties
    rb[5] = rb[2]; rb[9] = rb[2]; rb[n_experts - 1] = rb[0]
    rb[3] = 0x8000                                                   # -0.0 bias
    W = synth.MoeWeights(shape, rw, rb, W.gate_up_blocks, W.gate_up_scales, W.gate_up_bias, W.down_blocks,
                         W.down_scales, W.down_bias)
    T = 400
    hidden = synth.make_hidden(T, W, 7, min_gap=0.0)
    hidden[7] = 0                                                     # all logits = bias
    hidden[8] = 0x8000                                                # -0.0 everywhere
    layer = make_layer(shape, W, T)
    ridx, rwt = oracle.route(hidden, W.router_w, W.router_b, 4)
    results = {}
    for mma in (1, 0):
        layer.set_option("router_mma", mma)
        out, idx, w = run_device(layer, hidden)
        results[mma] = idx
        # tokens whose top-5 logits are well separated or exactly tied must match the oracle
        lg = oracle.route(hidden, W.router_w, W.router_b, 4, want_logits=True)[2].astype(np.float64)
        srt = -np.sort(-lg, axis=1)[:, :5]
        gaps = srt[:, :-1] - srt[:, 1:]
        safe = ((gaps > 1e-4) | (gaps == 0)).all(axis=1)
        assert safe.sum() > T // 2
        np.testing.assert_array_equal(idx[safe], ridx[safe], err_msg=f"router_mma={mma}")
        np.testing.assert_allclose(w[safe], rwt[safe], rtol=0, atol=2e-6)
    np.testing.assert_array_equal(results[1][[7, 8]], results[0][[7, 8]])
    layer.set_option("router_mma", 1)
    layer.close()


def test_graph_replay_matches_eager(full20b):
    """The third call with the same device buffers replays a captured CUDA graph; it must give
    the same bits as the eager launch sequence, also after the input buffer's contents change."""
    torch = torch_cuda()
    shape, W, layer = full20b
    lb = synth.zipf_logit_bias(shape.n_experts)
    d_lb = torch.from_numpy(lb).cuda()
    h = torch.empty((24, shape.hidden), dtype=torch.int16, device="cuda")
    out = torch.empty((24, shape.hidden), dtype=torch.float32, device="cuda")
    results = []
    for stream in (0, 0, 0, 1, 1):
        hidden = synth.make_hidden(24, W, 9, logit_bias=lb, stream=stream)
        h.copy_(torch.from_numpy(hidden.view(np.int16)))
        layer.run(h, logit_bias=d_lb, out=out)
        torch.cuda.synchronize()
        results.append(out.cpu().numpy().copy())
    layer.set_option("use_graphs", 0)
    layer.run(h, logit_bias=d_lb, out=out)
    torch.cuda.synchronize()
    eager = out.cpu().numpy()
    layer.set_option("use_graphs", 1)
    np.testing.assert_array_equal(results[0], results[1])
    np.testing.assert_array_equal(results[1], results[2])
    np.testing.assert_array_equal(results[3], results[4])
    np.testing.assert_array_equal(results[4], eager)
    assert not np.array_equal(results[2], results[3])


def test_config2_prefill_full_size(full20b):
    """T=4096, uniform routing (the prefill configuration): routing exact for every token,
    oracle on a token sample, finite outputs, counts add up."""
    shape, W, _ = full20b
    layer = make_layer(shape, W, max_tokens=4096)
    hidden = synth.make_hidden(4096, W, 6)
    toks = np.arange(5, 4096, 257, dtype=np.int32)
    out, _ = check_against_oracle(layer, W, hidden, tokens=toks, what="T=4096")
    assert np.isfinite(out).all()
    count = layer.read_dispatch()[0]
    assert count.sum() == 4096 * 4 and count.min() > 256
    layer.close()


def test_config4_shape_128_experts():
    """The 128-expert shape on one GPU (no sharding): T=300, oracle on a token sample."""
    shape = synth.MoeShape(n_experts=128)
    W = synth.make_weights(shape, 2)
    layer = make_layer(shape, W, max_tokens=300)
    hidden = synth.make_hidden(300, W, 2)
    toks = np.arange(0, 300, 23, dtype=np.int32)
    check_against_oracle(layer, W, hidden, tokens=toks, what="E=128")
    layer.close()


def test_packed_fp4_decode_option(full20b):
    """Option mx4=1: decode passes on tcgen05.mma.kind::mxf4 (packed 4-bit weights in shared
    memory, six e2m1 terms per activation).  Routing stays exact; outputs meet the contract."""
    shape, W, layer = full20b
    layer.set_option("mx4", 1)
    try:
        lb = synth.zipf_logit_bias(shape.n_experts)
        for T, seed in ((64, 12), (3, 13)):
            hidden = synth.make_hidden(T, W, seed, logit_bias=lb)
            check_against_oracle(layer, W, hidden, logit_bias=lb, what=f"mx4 T={T}")
    finally:
        layer.set_option("mx4", 0)


def test_fused_router_dispatch_equals_separate_kernels(full20b):
    """Option fuse_dispatch: the last router CTA running the dispatch gives the same routing,
    dispatch arrays and outputs (bit for bit) as the separate dispatch kernel."""
    shape, W, layer = full20b
    lb = synth.zipf_logit_bias(shape.n_experts)
    layer.set_option("decode_fused", 0)     # both arms on the multi-kernel path (the one-launch decode pass has no dispatch kernel)
    try:
        for T, seed in ((64, 41), (8, 42), (1, 43), (17, 44)):
            hidden = synth.make_hidden(T, W, seed, logit_bias=lb)
            layer.set_option("fuse_dispatch", 1)
            out1, _ = check_against_oracle(layer, W, hidden, logit_bias=lb, what=f"fused T={T}")
            d1 = layer.read_dispatch()
            layer.set_option("fuse_dispatch", 0)
            out0, _ = check_against_oracle(layer, W, hidden, logit_bias=lb, what=f"separate T={T}")
            d0 = layer.read_dispatch()
            np.testing.assert_array_equal(out1, out0)
            for a, b in zip(d1, d0):
                np.testing.assert_array_equal(a, b)
    finally:
        layer.set_option("fuse_dispatch", 0)
        layer.set_option("decode_fused", 1)


def test_pipelined_host_batches_equal_blocking_calls(full20b):
    """neon_moe_forward_host_batches: same results as one blocking host call per batch."""
    import torch
    shape, W, layer = full20b
    T, n = 16, 7
    hs = [torch.from_numpy(synth.make_hidden(T, W, 60 + i).view(np.int16)).pin_memory() for i in range(n)]
    outs = [torch.zeros((T, shape.hidden), dtype=torch.float32).pin_memory() for _ in range(n)]
    layer.run_host_batches([h.data_ptr() for h in hs], T, None, [o.data_ptr() for o in outs])
    for h, o in zip(hs, outs):
        ref = layer.run_host(h.numpy().view(np.uint16))
        ref = ref[0] if isinstance(ref, tuple) else ref
        np.testing.assert_array_equal(o.numpy(), ref)
    assert layer.status() == 0


def test_mma_rate_measurement():
    """The in-library ceiling of the block-scaled MMA instructions: plausible and monotone in N."""
    from neonengine_b200 import mma_rate
    r64 = mma_rate.measure("mxf8f6f4", 64, 2048)
    r256 = mma_rate.measure("mxf8f6f4", 256, 2048)
    r4 = mma_rate.measure("mxf4", 256, 2048)
    for r in (r64, r256, r4):
        assert r["cycles_per_mma"] > 8 and 50.0 < r["tflops"] < 20000.0
    assert r256["tflops"] > r64["tflops"]          # larger N amortises the weight-operand read
    assert r4["tflops"] > 0.9 * r256["tflops"]     # packed 4-bit operands are at least as fast
    lib = __import__("neonengine_b200._lib", fromlist=["load"]).load()
    import ctypes
    ms, cyc = ctypes.c_double(), ctypes.c_int64()
    assert lib.neon_moe_mma_rate(0, 0, 100, 16, ctypes.byref(ms), ctypes.byref(cyc)) == 1   # n not a multiple of 16


def test_tma_copy_rate_measurement():
    """The library's copy-rate probe: one SM's TMA unit streaming weight boxes with no consumer.  From a buffer
    that stays in L2 a box pair lands every few hundred clocks; from a buffer far larger than L2 the whole GPU
    runs at HBM pace; the scale-copy variant of the MMA probe costs a few clocks per instruction more."""
    from neonengine_b200 import mma_rate
    l2 = mma_rate.tma_copy_rate(False, 4, 8, 1024)
    hbm = mma_rate.tma_copy_rate(False, 4, 1024, 1024)
    packed = mma_rate.tma_copy_rate(True, 4, 8, 1024)
    assert 20.0 < l2["bytes_per_cycle_per_sm"] < 128.0
    assert 3000.0 < hbm["gbs"] < 9000.0
    assert hbm["gbs"] < l2["gbs"]
    assert 0.5 < packed["bytes_per_cycle_per_sm"] / l2["bytes_per_cycle_per_sm"] < 2.0
    plain = mma_rate.measure("mxf8f6f4", 32, 2048)
    with_sf = mma_rate.measure("mxf8f6f4+sf", 32, 2048)
    assert plain["cycles_per_mma"] <= with_sf["cycles_per_mma"] < 2 * plain["cycles_per_mma"]
    lib = __import__("neonengine_b200._lib", fromlist=["load"]).load()
    import ctypes
    ms, cyc = ctypes.c_double(), ctypes.c_int64()
    assert lib.neon_moe_tma_rate(0, 0, 7, 8 << 20, 16, ctypes.byref(ms), ctypes.byref(cyc)) == 1   # too many stages


@pytest.mark.parametrize("T,sliced", [(1, 1), (2, 1), (3, 1), (4, 1), (1, 0), (2, 0), (4, 0), (7, 1), (8, 1)])
def test_one_launch_decode_pass(full20b, T, sliced):
    """Passes of at most 8 tokens run as ONE cooperative kernel (router, both expert products,
    SwiGLU and combine; no dispatch pass): up to 4 tokens sliced by intermediate channel (sliced = 1),
    above that - or with option decode_sliced 0 - cut into equal runs of K chunks.  Routing and the
    dispatch arrays it reports are bit-exact against the oracle, outputs within the contract; it
    launches exactly one kernel; two runs give the same bits; and the multi-kernel path agrees
    within the contract.  The two kernels share their pass counters, so the cases also check that
    they can alternate."""
    shape, W, layer = full20b
    lb = synth.zipf_logit_bias(shape.n_experts) if T in (4, 8) else None
    hidden = synth.make_hidden(T, W, 70 + T, logit_bias=lb)
    layer.set_option("use_graphs", 0)
    layer.set_option("decode_fused_tokens", 8)      # by default only single-token passes take the one-launch kernel
    layer.set_option("decode_sliced", sliced)
    try:
        before = layer.launch_count
        out, _ = check_against_oracle(layer, W, hidden, logit_bias=lb, what=f"one-launch T={T}")
        assert layer.launch_count - before == 1
        again = run_device(layer, hidden, lb)[0]
        np.testing.assert_array_equal(again, out)
        layer.set_option("decode_fused", 0)
        before = layer.launch_count
        multi = run_device(layer, hidden, lb)[0]
        assert layer.launch_count - before > 1
        assert_close(out, multi, f"one-launch vs multi-kernel T={T}")
        assert layer.status() == 0
    finally:
        layer.set_option("decode_fused", 1)
        layer.set_option("decode_sliced", 0)
        layer.set_option("decode_fused_tokens", 1)
        layer.set_option("use_graphs", 1)


@pytest.mark.parametrize("sliced", [1, 0])
def test_one_launch_decode_bounded_wait_reports_and_recovers(full20b, sliced):
    """Failure detection without a GPU fault: a test hook makes the kernel's first wait expect one
    arrival more than the grid can deliver.  Every CTA gives up after the (shortened) limit, the
    pass returns, the status word names the wait, and the next pass is correct again.  Both
    one-launch kernels."""
    shape, W, layer = full20b
    hidden = synth.make_hidden(2, W, 90)
    layer.set_option("use_graphs", 0)
    layer.set_option("decode_fused_tokens", 8)
    layer.set_option("decode_sliced", sliced)
    try:
        layer.set_option("decode_wait_limit", 100_000_000)   # ~50 ms of SM clocks
        layer.set_option("decode_stall_test", 1)
        run_device(layer, hidden)
        assert layer.status() == 7                            # code of the router-completion wait
        layer.set_option("decode_stall_test", 0)
        layer.set_option("decode_wait_limit", 400_000_000)
        check_against_oracle(layer, W, hidden, what="after a timed-out pass")
    finally:
        layer.set_option("decode_stall_test", 0)
        layer.set_option("decode_sliced", 0)
        layer.set_option("decode_fused_tokens", 1)
        layer.set_option("use_graphs", 1)


def test_mxf4_prefill_against_the_quantisation_aware_oracle(full20b, capsys):
    """Option mxf4_prefill: 128-token tiles on tcgen05.mma.kind::mxf4 with the activations quantised to
    MXFP4 (blocks of 32, E8M0 scale 2^(floor(log2 amax) - 2), nearest e2m1, ties to even) - the rule
    of the oracle's quant_act mode.  Routing stays exact.  Against the quantisation-aware oracle the
    outputs agree to accumulation noise except where a SwiGLU value sits within float rounding of
    a quantisation boundary and the two sides round it to different codes (one code step of one
    activation moves an output by up to ~0.5): so the mean relative error must meet the contract,
    and at most 1 output in 1000 may miss the absolute bound.  Against the plain oracle this path
    is, by construction, far outside the contract (4-bit activations): that error is printed."""
    shape, W, _ = full20b
    T = 1024
    layer = make_layer(shape, W, max_tokens=T)
    layer.set_option("mxf4_prefill", 1)
    hidden = synth.make_hidden(T, W, 8)
    out, idx, w = run_device(layer, hidden)
    ridx, rw = oracle.route(hidden, W.router_w, W.router_b, shape.top_k)
    np.testing.assert_array_equal(idx, ridx)
    toks = np.arange(7, T, 97, dtype=np.int32)
    ref_q = oracle.experts(hidden, ridx, rw, W, tokens=toks, quant_act=True)
    ref = oracle.experts(hidden, ridx, rw, W, tokens=toks)
    got = out[toks].astype(np.float64)
    err_q = np.abs(got - ref_q)
    mean_rel_q = err_q.mean() / np.abs(ref_q).mean()
    frac_over = (err_q > 2e-2).mean()
    mean_rel_plain = np.abs(got - ref).mean() / np.abs(ref).mean()
    with capsys.disabled():
        print(f"\n[mxf4 prefill] vs quantisation-aware oracle: mean_rel {mean_rel_q:.3e}, max_abs {err_q.max():.3e}, "
              f"outputs over 2e-2: {frac_over:.2e}; vs plain oracle: mean_rel {mean_rel_plain:.3e}, "
              f"max_abs {np.abs(got - ref).max():.3e}")
    assert layer.status() == 0
    assert mean_rel_q <= 5e-3 and frac_over <= 1e-3, (mean_rel_q, frac_over)
    assert mean_rel_plain > 5e-3          # 4-bit activations cannot meet the contract against the unquantised result
    layer.close()


@pytest.mark.parametrize("T", [3, 17, 64, 200, 384])
def test_two_sm_mma_decode_tiles(full20b, T):
    """Option pair_mma: decode tiles on clusters of two CTAs and two-SM MMAs (tcgen05 cta_group::2).  Same
    routing, dispatch and - the same products accumulated in the same order - the same output bits as the
    one-CTA kernel; checked against the oracle as well.  T=3 and 17 leave the second tile of odd tile counts
    and ragged token tiles to both CTAs of a pair."""
    shape, W, layer = full20b
    lb = synth.zipf_logit_bias(shape.n_experts) if T == 64 else None
    hidden = synth.make_hidden(T, W, 200 + T, logit_bias=lb)
    toks = None if T <= 64 else np.arange(1, T, 23, dtype=np.int32)
    layer.set_option("decode_fused", 0)
    layer.set_option("pair_mma", 0)
    layer.set_option("tile_tokens", 0 if T <= 16 else 32)   # 32-token tiles also where 128-token ones are the default
    try:
        ref = run_device(layer, hidden, lb)[0]
        layer.set_option("pair_mma", 1)
        out, _ = check_against_oracle(layer, W, hidden, logit_bias=lb, tokens=toks, what=f"pair_mma T={T}")
        np.testing.assert_array_equal(out, ref)
    finally:
        layer.set_option("pair_mma", 2)
        layer.set_option("tile_tokens", 0)
        layer.set_option("decode_fused", 1)


@pytest.mark.parametrize("T", [385, 700, 4096])
def test_two_sm_mma_prefill_tiles(full20b_prefill, T):
    """128-token tiles on CTA pairs (option pair_prefill, the default): each CTA streams its own weight tile
    and half of the token rows, the leader issues M = 256 instructions with the tile's own per-row block
    scales.  Same products in the same order as the one-CTA kernel: identical output bits; checked against the
    oracle as well.  T = 385 and 700 leave ragged last tiles (N not a multiple of 128)."""
    shape, W, layer = full20b_prefill
    hidden = synth.make_hidden(T, W, 400 + T)
    toks = np.arange(1, T, max(1, T // 12), dtype=np.int32)
    layer.set_option("pair_prefill", 0)
    try:
        ref = run_device(layer, hidden, None)[0]
        layer.set_option("pair_prefill", 1)
        out, _ = check_against_oracle(layer, W, hidden, tokens=toks, what=f"pair_prefill T={T}")
        np.testing.assert_array_equal(out, ref)
        assert layer.status() == 0
    finally:
        layer.set_option("pair_prefill", 1)


@pytest.mark.parametrize("T", [257, 700, 4096])
def test_many_cta_dispatch_equals_one_cta(full20b_prefill, T):
    """Passes of more than 1024 entries sort their entries on one CTA per 1024 entries (counts per chunk, one
    scan by the CTA that finishes last, placement by every CTA).  Counts, offsets, the stable permutation and
    its inverse equal the one-CTA kernel's and the oracle's; outputs are bit-identical."""
    shape, W, layer = full20b_prefill
    hidden = synth.make_hidden(T, W, 500 + T)
    layer.set_option("dispatch_multi", 0)
    try:
        ref = run_device(layer, hidden, None)[0]
        d_ref = layer.read_dispatch()
        layer.set_option("dispatch_multi", 1)
        out = run_device(layer, hidden, None)[0]
        d_new = layer.read_dispatch()
        for a, b in zip(d_ref, d_new):
            np.testing.assert_array_equal(a, b)
        np.testing.assert_array_equal(out, ref)
        again = run_device(layer, hidden, None)[0]      # the arrival counter was left at zero
        np.testing.assert_array_equal(again, ref)
        ridx, _ = oracle.route(hidden, W.router_w, W.router_b, shape.top_k)
        count, offset, perm, inv = oracle.dispatch(ridx, shape.n_experts)
        np.testing.assert_array_equal(d_new[0], count)
        np.testing.assert_array_equal(d_new[2], perm)
        assert layer.status() == 0
    finally:
        layer.set_option("dispatch_multi", 1)


def test_two_sm_mma_instruction_self_check():
    """The library's self-check of the two-SM instruction form: M = 256 splits by CTA, the N operand is the
    concatenation of the two CTAs' halves, the multicast commit reaches both CTAs (no timeout)."""
    import ctypes
    lib = __import__("neonengine_b200._lib", fromlist=["load"]).load()
    for n, chunks in ((64, 3), (32, 1)):
        d = np.zeros((2, 4, 4), np.float32)
        addr = np.zeros(2, np.uint32)
        cyc = ctypes.c_int64()
        assert lib.neon_moe_mma_pair_probe(0, n, chunks, d.ctypes.data, addr.ctypes.data, ctypes.byref(cyc)) == 0
        want = chunks * 128.0 * np.array([1, 1, 2, 2], np.float32)
        np.testing.assert_array_equal(d[0], np.tile(want, (4, 1)))
        np.testing.assert_array_equal(d[1], np.tile(0.5 * want, (4, 1)))
        assert addr[0] == addr[1] and cyc.value > 0
    assert lib.neon_moe_mma_pair_probe(0, 48, 1, d.ctypes.data, addr.ctypes.data, ctypes.byref(cyc)) == 1
