"""Expert parallelism on GPUs: two ranks (one process per GPU) run `neon_moe_forward_ep`
through the C ABI and must reproduce the single-process CPU oracle: routing bit-exact,
outputs within the contract tolerance.  Skipped when fewer than two GPUs are visible."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    import oracle
    from helpers import assert_close
    from neonengine_b200 import synth
    from neonengine_b200.moe_layer_system import MoeLayerSystem
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    shape = synth.MoeShape(hidden=2880, inter=2880, n_experts=8, top_k=4)
    full = synth.make_weights(shape, 31)
    nl = shape.n_experts // world
    layer = MoeLayerSystem(shape, full.slice_experts(rank * nl, (rank + 1) * nl), max_tokens=T + world,
                           device=rank, ep_rank=rank, ep_size=world)
    ids = [MoeLayerSystem.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    layer.ep_init(ids[0])
    for step in range(2):                       # two passes: buffers are reused
        hidden = synth.make_hidden(T + rank, full, 31, stream=10 * step + rank)   # ragged T across ranks
        h = torch.from_numpy(hidden.view(np.int16)).cuda()
        out, idx, w = layer.run_ep(h, want_routing=True)
        torch.cuda.synchronize()
        ref, ridx, rw = oracle.moe_forward(hidden, full)
        np.testing.assert_array_equal(idx.cpu().numpy(), ridx)
        assert_close(out.cpu().numpy(), ref, f"rank {rank} step {step}")
        assert layer.status() == 0
    dist.barrier()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    layer.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("T", [6, 200])
def test_two_gpu_expert_parallel_matches_oracle(tmp_path, T):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), T, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
