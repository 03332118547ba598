"""Expert parallelism on the CPU: two gloo ranks run the exchange the library plans
(`neon_moe_ep_plan`, a host-only C-ABI call) with the CPU oracle standing in for the local
expert products, and must reproduce the single-process oracle.  This covers the N > 1 host
logic: who sends which rows to whom, in which order, and how a receiver recovers each
row's expert from the gathered histograms alone."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _exchange(rows_by_peer, recv_counts, width, dtype, rank, world):
    """all-to-all-v with point-to-point gloo ops; returns the concatenated received rows."""
    recv = [torch.empty((int(recv_counts[r]), width), dtype=dtype) for r in range(world)]
    reqs = []
    for r in range(world):
        if r == rank:
            recv[r].copy_(rows_by_peer[r])
            continue
        reqs.append(dist.isend(rows_by_peer[r].contiguous(), r))
        reqs.append(dist.irecv(recv[r], r))
    for q in reqs:
        q.wait()
    return torch.cat(recv, 0)


def _worker(rank, world, port, T, seed, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from neonengine_b200 import synth
    from neonengine_b200.moe_layer_system import ep_plan
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shape = synth.MoeShape(hidden=64, inter=64, n_experts=8, top_k=4)
    full = synth.make_weights(shape, seed)
    nl = shape.n_experts // world
    mine = synth.make_weights(shape, seed, experts=(rank * nl, (rank + 1) * nl))
    hidden = synth.make_hidden(T + rank, full, seed, stream=rank)          # ragged: ranks hold different T
    idx, w = oracle.route(hidden, full.router_w, full.router_b, shape.top_k)
    count, offset, perm, inv = oracle.dispatch(idx, shape.n_experts)
    gathered = [torch.zeros(shape.n_experts, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(count))
    all_counts = torch.stack(gathered).numpy()
    send_rows, send_off, recv_rows, recv_off, row_expert = ep_plan(all_counts, rank)
    assert send_rows.sum() == idx.size and recv_rows.sum() == row_expert.size
    xsend = torch.from_numpy(hidden.astype(np.int32))[torch.from_numpy(perm // shape.top_k)]
    parts = [xsend[send_off[r]:send_off[r] + send_rows[r]] for r in range(world)]
    xrecv = _exchange(parts, recv_rows, shape.hidden, torch.int32, rank, world).numpy().astype(np.uint16)
    # local experts: one slot per received row, unit weight
    R = xrecv.shape[0]
    y = oracle.experts(xrecv, row_expert.reshape(R, 1) + rank * nl, np.ones((R, 1), np.float32), mine, e_lo=rank * nl) \
        if R else np.zeros((0, shape.hidden), np.float32)
    back = [torch.from_numpy(y[recv_off[r]:recv_off[r] + recv_rows[r]]) for r in range(world)]
    yrecv = _exchange(back, send_rows, shape.hidden, torch.float32, rank, world).numpy()
    out = np.zeros((hidden.shape[0], shape.hidden), np.float64)
    for t in range(hidden.shape[0]):
        for s in range(shape.top_k):
            out[t] += np.float64(w[t, s]) * yrecv[inv[t * shape.top_k + s]]
    ref, ridx, rw = oracle.moe_forward(hidden, full)
    np.testing.assert_array_equal(idx, ridx)
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-6)
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    dist.destroy_process_group()


@pytest.mark.parametrize("T", [5, 33])
def test_two_rank_exchange_matches_single_process(tmp_path, T):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), T, 17, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_plan_known_answer():
    sys.path.insert(0, ROOT)
    from neonengine_b200.moe_layer_system import ep_plan
    # 2 ranks, 4 experts (2 each).  rank 0 routes [3,0,2,1], rank 1 routes [1,1,0,5]
    counts = np.array([[3, 0, 2, 1], [1, 1, 0, 5]], np.int32)
    s, so, r, ro, re = ep_plan(counts, 0)
    assert s.tolist() == [3, 3] and so.tolist() == [0, 3]
    assert r.tolist() == [3, 2] and ro.tolist() == [0, 3]
    assert re.tolist() == [0, 0, 0, 0, 1]
    s, so, r, ro, re = ep_plan(counts, 1)
    assert s.tolist() == [2, 5] and r.tolist() == [3, 5]
    assert re.tolist() == [0, 0, 1, 1, 1, 1, 1, 1]
    with pytest.raises(RuntimeError):
        ep_plan(counts, 1, cap=4)     # would receive 8 rows


def test_capacity_verdict_is_the_same_on_every_rank():
    """A skewed four-rank histogram: rank 0 would receive more than its room while the other
    ranks' own totals fit.  The verdict is computed from the gathered histograms and names rank 0
    whichever rank evaluates it, so no rank posts an exchange that a peer has walked away from."""
    import ctypes
    sys.path.insert(0, ROOT)
    from neonengine_b200 import _lib
    from neonengine_b200.moe_layer_system import ep_plan
    lib = _lib.load()
    G, E, k, T = 4, 16, 4, 8
    counts = np.zeros((G, E), np.int32)
    counts[:, 0:4] = [12, 10, 6, 2]          # 30 of each rank's 32 entries go to rank 0's experts
    counts[:, 4] = 1
    counts[:, 8] = 1
    assert (counts.sum(1) == T * k).all()
    caps = np.full(G, 2 * T * k, np.int32)   # 64 rows each; rank 0 would get 120
    first = ctypes.c_int(-2)
    assert lib.neon_moe_ep_overflow(counts.ctypes.data, G, E, caps.ctypes.data, ctypes.byref(first)) == 0
    assert first.value == 0
    # the per-rank plan alone would let ranks 1..3 carry on: that is why it is not the verdict
    for r in (1, 2, 3):
        ep_plan(counts, r, cap=int(caps[r]))
    with pytest.raises(RuntimeError):
        ep_plan(counts, 0, cap=int(caps[0]))
    # halving every rank's token range halves the histogram: the halves fit
    half = counts // 2
    assert lib.neon_moe_ep_overflow(half.ctypes.data, G, E, caps.ctypes.data, ctypes.byref(first)) == 0
    assert first.value == -1
    # ranks with different capacities: the verdict uses each rank's own
    caps2 = np.array([200, 3, 200, 200], np.int32)
    assert lib.neon_moe_ep_overflow(counts.ctypes.data, G, E, caps2.ctypes.data, ctypes.byref(first)) == 0
    assert first.value == 1
    assert lib.neon_moe_ep_overflow(None, G, E, caps.ctypes.data, ctypes.byref(first)) == 1
