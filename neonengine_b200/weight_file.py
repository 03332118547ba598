"""Host side of the MoE weight-file format (layout in include/neon_moe.h).

``write_raw`` packs a :class:`MoeWeights` into a "raw" file (the tensors as
``neon_moe_set_weights`` takes them); ``read`` maps any weight file and returns its header and
sections as numpy views.  "Tiled" files are written by the library from a loaded handle
(``MoeLayerSystem.save_weights``) and can be inspected with ``read`` as well.
"""
from __future__ import annotations

import struct

import numpy as np

from .synth import MoeShape, MoeWeights

MAGIC = b"NMOEW1\0\0"
HEADER = struct.Struct("<8sII6iI5I")      # 64 bytes
SECTION = struct.Struct("<16sQQ")         # 32 bytes
RAW_SECTIONS = ("router_w", "router_b", "gu_blocks", "gu_scales", "gu_bias", "dn_blocks", "dn_scales", "dn_bias")


def _align(v: int) -> int:
    return (v + 255) & ~255


def write_raw(path: str, w: MoeWeights, expert_lo: int = 0) -> None:
    """Raw layout; ``w`` holds experts [expert_lo, expert_lo + n_local) and the full router."""
    s = w.shape
    arrays = [np.ascontiguousarray(a) for a in (w.router_w, w.router_b, w.gate_up_blocks, w.gate_up_scales, w.gate_up_bias,
                                                w.down_blocks, w.down_scales, w.down_bias)]
    n_local = arrays[2].shape[0]
    table, off = [], _align(HEADER.size + len(arrays) * SECTION.size)
    for name, a in zip(RAW_SECTIONS, arrays):
        table.append((name, off, a.nbytes))
        off = _align(off + a.nbytes)
    with open(path, "wb") as f:
        f.write(HEADER.pack(MAGIC, 1, 0, s.hidden, s.inter, s.n_experts, expert_lo, n_local, s.top_k, len(arrays), 0, 0, 0, 0, 0))
        for name, o, n in table:
            f.write(SECTION.pack(name.encode(), o, n))
        for (name, o, n), a in zip(table, arrays):
            f.seek(o)
            f.write(a.tobytes())
        f.truncate(off)  # zero padding up to the aligned end


def read(path: str):
    """Returns (header dict, {section name: uint8 memmap view})."""
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    magic, version, layout, hidden, inter, n_experts, expert_lo, n_local, top_k, n_sections, *_ = HEADER.unpack(bytes(mm[:HEADER.size]))
    if magic != MAGIC or version != 1:
        raise ValueError(f"{path} is not a version-1 weight file")
    header = dict(layout=layout, hidden=hidden, inter=inter, n_experts=n_experts, expert_lo=expert_lo, n_local=n_local, top_k=top_k)
    sections = {}
    for i in range(n_sections):
        o = HEADER.size + i * SECTION.size
        name, off, nbytes = SECTION.unpack(bytes(mm[o:o + SECTION.size]))
        if off + nbytes > mm.size:
            raise ValueError(f"{path} is truncated inside section {name!r}")
        sections[name.rstrip(b"\0").decode()] = mm[off:off + nbytes]
    return header, sections


def read_raw(path: str) -> MoeWeights:
    h, s = read(path)
    if h["layout"] != 0:
        raise ValueError("not a raw weight file")
    shape = MoeShape(hidden=h["hidden"], inter=h["inter"], n_experts=h["n_experts"], top_k=h["top_k"])
    E, EL, H, I = h["n_experts"], h["n_local"], h["hidden"], h["inter"]
    u16 = lambda a, dims: np.frombuffer(a, np.uint16).reshape(dims)  # noqa: E731
    return MoeWeights(shape, u16(s["router_w"], (E, H)), u16(s["router_b"], (E,)),
                      np.asarray(s["gu_blocks"]).reshape(EL, 2 * I, H // 2), np.asarray(s["gu_scales"]).reshape(EL, 2 * I, H // 32),
                      u16(s["gu_bias"], (EL, 2 * I)), np.asarray(s["dn_blocks"]).reshape(EL, H, I // 2),
                      np.asarray(s["dn_scales"]).reshape(EL, H, I // 32), u16(s["dn_bias"], (EL, H)))
