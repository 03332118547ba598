"""Weight-file format (include/neon_moe.h): host packer round trip (CPU), and on the GPU the
library's loader for both layouts against neon_moe_set_weights, plus the "tiled" file's bytes
against an independent numpy restatement of the tensor-core layout."""
import os

import numpy as np
import pytest

from neonengine_b200 import synth, weight_file

SHAPE = synth.MoeShape(hidden=256, inter=192, n_experts=8, top_k=4)


def tc_layout_numpy(blocks, scales, gate_up):
    """Independent restatement of the tensor-core layout: nibbles box by box
    [E][m_tiles][k_chunks][128 rows][64 B] (rows and K padded with zeros), gate_up rows permuted so
    that tile row r = 32q + l of tile m holds channel 64m + 16q + l%16, gate (l < 16) or linear;
    scales as 512-byte atoms, byte (r%32)*16 + (r/32)*4 + kb, pads = 127."""
    E, rows, kb2 = blocks.shape
    K = kb2 * 2
    n_chunks, m_tiles = (K + 127) // 128, (rows + 127) // 128
    tiles = np.zeros((E, m_tiles, n_chunks, 128, 64), np.uint8)
    sfa = np.full((E, m_tiles, n_chunks, 512), 127, np.uint8)
    for m in range(m_tiles):
        for r in range(128):
            row = 128 * m + r
            if row >= rows:
                continue
            if gate_up:
                q, l = (r >> 5) & 3, r & 31
                src = 2 * (64 * m + 16 * q + (l & 15)) + (l >> 4)
            else:
                src = row
            for c in range(n_chunks):
                nb = min(64, kb2 - c * 64)
                if nb > 0:
                    tiles[:, m, c, r, :nb] = blocks[:, src, c * 64:c * 64 + nb]
                for kb in range(4):
                    blk = 4 * c + kb
                    if blk < K // 32:
                        sfa[:, m, c, (r % 32) * 16 + (r // 32) * 4 + kb] = scales[:, src, blk]
    return tiles.reshape(-1), sfa.reshape(-1)


def test_raw_file_round_trip(tmp_path):
    W = synth.make_weights(SHAPE, 3)
    path = tmp_path / "layer.nmoe"
    weight_file.write_raw(str(path), W)
    header, sections = weight_file.read(str(path))
    assert header == dict(layout=0, hidden=256, inter=192, n_experts=8, expert_lo=0, n_local=8, top_k=4)
    assert set(sections) == set(weight_file.RAW_SECTIONS)
    back = weight_file.read_raw(str(path))
    for name in ("router_w", "router_b", "gate_up_blocks", "gate_up_scales", "gate_up_bias", "down_blocks", "down_scales",
                 "down_bias"):
        np.testing.assert_array_equal(getattr(back, name), getattr(W, name))
    assert os.path.getsize(path) % 256 == 0
    # an expert-parallel shard file
    shard = W.slice_experts(4, 8)
    weight_file.write_raw(str(tmp_path / "shard.nmoe"), shard, expert_lo=4)
    h2, _ = weight_file.read(str(tmp_path / "shard.nmoe"))
    assert h2["expert_lo"] == 4 and h2["n_local"] == 4
    with open(tmp_path / "bad.nmoe", "wb") as f:
        f.write(b"not a weight file" * 8)
    with pytest.raises(ValueError):
        weight_file.read(str(tmp_path / "bad.nmoe"))


@pytest.mark.gpu
def test_loader_matches_set_weights_and_tiled_bytes(tmp_path):
    import torch
    from neonengine_b200.moe_layer_system import MoeLayerSystem
    W = synth.make_weights(SHAPE, 3)
    hidden = synth.make_hidden(16, W, 5)
    h = torch.from_numpy(hidden.view(np.int16)).cuda()
    a = MoeLayerSystem(SHAPE, W, max_tokens=16)
    ref = a.run(h).cpu().numpy()
    raw, tiled = str(tmp_path / "raw.nmoe"), str(tmp_path / "tiled.nmoe")
    weight_file.write_raw(raw, W)
    a.save_weights(tiled)
    # the tiled file holds exactly the restated tensor-core layout
    header, sec = weight_file.read(tiled)
    assert header["layout"] == 1
    gt, gs = tc_layout_numpy(W.gate_up_blocks, W.gate_up_scales, True)
    dt, ds = tc_layout_numpy(W.down_blocks, W.down_scales, False)
    np.testing.assert_array_equal(np.asarray(sec["gu_tiles"]), gt)
    np.testing.assert_array_equal(np.asarray(sec["gu_sfa"]), gs)
    np.testing.assert_array_equal(np.asarray(sec["dn_tiles"]), dt)
    np.testing.assert_array_equal(np.asarray(sec["dn_sfa"]), ds)
    np.testing.assert_array_equal(np.frombuffer(sec["router_w"], np.uint16).reshape(W.router_w.shape), W.router_w)
    for path in (raw, tiled):
        b = MoeLayerSystem(SHAPE, None, max_tokens=16)
        with pytest.raises(RuntimeError, match="set_weights"):
            b.run(h)
        b.load_weights_file(path)
        np.testing.assert_array_equal(b.run(h).cpu().numpy(), ref)
        # only the tensor-core layout is in a file; the mma.sync kernels' layout is rebuilt from it on
        # request and must then serve the same weights
        with pytest.raises(RuntimeError, match="mma16_layout"):
            b.run_static(h)
        b.set_option("path", 1)
        via_mma = b.run(h).cpu().numpy()
        a.set_option("path", 1)
        np.testing.assert_array_equal(via_mma, a.run(h).cpu().numpy())
        a.set_option("path", 2)
        b.close()
    # refusals: wrong shape, truncated file, missing file
    other = MoeLayerSystem(synth.MoeShape(hidden=256, inter=128, n_experts=8, top_k=4), None, max_tokens=4)
    with pytest.raises(RuntimeError, match="expects"):
        other.load_weights_file(raw)
    with open(raw, "rb") as f:
        data = f.read()
    with open(tmp_path / "cut.nmoe", "wb") as f:
        f.write(data[:len(data) // 2])
    c = MoeLayerSystem(SHAPE, None, max_tokens=4)
    with pytest.raises(RuntimeError, match="truncated"):
        c.load_weights_file(str(tmp_path / "cut.nmoe"))
    with pytest.raises(RuntimeError, match="cannot open"):
        c.load_weights_file(str(tmp_path / "missing.nmoe"))
    a.close(); other.close(); c.close()
