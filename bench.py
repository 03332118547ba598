#!/usr/bin/env python
"""Benchmark of the gpt-oss-shaped MoE layer (tokens/s) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg0|cfg1|cfg2|cfg3|cfg4|water|svgf|pt] [--impl reference]

A step is one pass of the MoE layer over one batch of seeded synthetic hidden states.
Default workload at one GPU is the batched-decode configuration (T=64 tokens, Zipf-skewed
routing, gpt-oss-20b shapes); batches rotate and the 424 MB of expert weights exceed the
126 MB L2, so every step streams its weights from HBM.  With N > 1 GPUs (torchrun) the default
is the 128-expert configuration, expert-parallel: experts sharded over the ranks, token rows
exchanged by all-to-all over NVLink (NCCL), 8192 tokens per GPU (weak scaling).

One JSON line is printed by rank 0:
  value     tokens/s with inputs resident in HBM (CUDA events on the launching stream)
  e2e       tokens/s through the host-buffer C-ABI call (pinned host in/out, copies timed)
  roofline  achieved HBM GB/s of the dominant kernel (gate_up expert product) = its
            algorithmic bytes / its mean launch duration, against the measured copy peak
  cpu_baseline  the CPU oracle on a bounded sample of the same workload, on the host cores
`--workload cfg3` runs the whole gpt-oss-20b-shaped decoder (24 layers, decode batch 8, 4096-token
K/V cache, 201088-token vocabulary; one step = one new token per sequence, tokens fed back).
`--workload water` runs the reference engine's own FLIP water step (8000 particles, 99x37x44 cells,
4 separation sub-steps, 50 Jacobi iterations per step) and reports simulation steps/s; its CPU arm
is the reference shader itself compiled for the host (oracle/_ref) when present, else the restatement.
`--workload svgf` runs the reference engine's denoiser (temporal accumulation + 3 a-trous passes) on
1920x1080 frames of a seeded synthetic scene and reports frames/s; CPU arm as for the water step.
`--impl reference` times the CPU oracle alone (the nominal reference engine has no
implementation of this path; the oracle is its stand-in on the host cores).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from neonengine_b200 import synth  # noqa: E402

FALLBACK_HBM_GBS = 6650.0

WORKLOADS = {
    # name: (T, n_experts, zipf, description)
    "cfg0": (1, 32, False, "gpt-oss-20b MoE layer, decode T=1"),
    "cfg1": (64, 32, True, "gpt-oss-20b MoE layer, batched decode T=64, Zipf(1.1) router bias"),
    "cfg2": (4096, 32, False, "gpt-oss-20b MoE layer, prefill T=4096, uniform routing"),
    "cfg3": (8, 32, False, "gpt-oss-20b-shaped decoder, 24 layers, decode batch 8, 4096-token bf16 K/V cache, "
                           "vocabulary 201088, random-init weights"),
    "water": (0, 0, False, "NeonEngine FLIP water step: 8000 particles, 99x37x44 cells, 4 separation sub-steps, "
                           "50 pressure Jacobi iterations, dt 1/500"),
    "svgf": (0, 0, False, "NeonEngine denoiser: temporal accumulation + 3 a-trous passes of one 1920x1080 frame "
                          "(rgba32f G-buffer, rgba16f history, rgba8 image), seeded synthetic scene"),
    "pt": (0, 0, False, "NeonEngine path tracer: Cornell box with 50 sphere lights (11248 triangles), 800x600, one sample per "
                        "pixel, at most 3 bounces with next-event estimation (raygen.rgen + closesthit.rchit + miss shaders)"),
    "cfg4": (8192, 128, False, "gpt-oss-120b-shaped MoE layer, 128 experts, T=8192 tokens per GPU, uniform routing, "
                               "experts sharded over the GPUs (expert parallel) when more than one"),
}


_JSON_FD = None


def claim_stdout():
    """Libraries (NCCL's version banner, for one) write to file descriptor 1.  From here on fd 1 is
    stderr for everybody; the one JSON line goes to the original stdout through emit()."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, device_index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
        self.period = period_s

    def _run(self):
        nv = self._nv
        names = {
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_batches(T, W, zipf, n_batches, base_stream=0):
    lb = synth.zipf_logit_bias(W.shape.n_experts) if zipf else None
    return [synth.make_hidden(T, W, 0, logit_bias=lb, stream=base_stream + i) for i in range(n_batches)], lb


def cpu_steps(W, batches, lb, seconds_budget, max_tokens_per_step=None):
    """Times the CPU oracle on whole batches (or their first max_tokens_per_step tokens)."""
    import oracle
    oracle.lib()
    done_tokens, t_total, steps = 0, 0.0, 0
    while t_total < seconds_budget and steps < 64:
        hid = batches[steps % len(batches)]
        if max_tokens_per_step:
            hid = hid[:max_tokens_per_step]
        t0 = time.perf_counter()
        oracle.moe_forward(hid, W, logit_bias=lb)
        t_total += time.perf_counter() - t0
        done_tokens += hid.shape[0]
        steps += 1
    return done_tokens / t_total, steps, oracle.n_threads()


def run_reference(args, rank):
    """CPU arm: the oracle on the host cores, same workload, bounded sample per step."""
    if rank != 0:
        return
    T, E, zipf, desc = WORKLOADS[args.workload]
    shape = synth.MoeShape(n_experts=E)
    W = synth.make_weights(shape, 0)
    sample_T = min(T, 64)
    batches, lb = make_batches(sample_T, W, zipf, 4)
    import oracle
    oracle.lib()
    for i in range(min(args.warmup, 1)):
        oracle.moe_forward(batches[0], W, logit_bias=lb)
    t0 = time.perf_counter()
    for i in range(args.steps):
        oracle.moe_forward(batches[i % len(batches)], W, logit_bias=lb)
    dt = time.perf_counter() - t0
    tps = args.steps * sample_T / dt
    cores = oracle.n_threads()
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "tokens_per_step": sample_T},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": f"{args.steps} steps of {sample_T} tokens (CPU oracle, OpenMP, fp64 accumulate)"},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def decoder_cpu_sample(vocab_slice=8192):
    """Times the CPU restatement of one decode step on a bounded sample: ONE layer at the real
    widths (batch 8, 4096-token cache) plus a `vocab_slice`-row slice of the unembedding, and
    extrapolates to 24 layers and the whole vocabulary.  Returns (tokens/s, cores, description)."""
    import dataclasses
    import oracle
    from oracle import decoder_oracle as dor
    from neonengine_b200.decoder_synth import DecoderShape, make_decoder_weights, make_kv
    oracle.lib()
    full = DecoderShape()
    shape = dataclasses.replace(full, n_layers=1, vocab=vocab_slice)
    B, ctx = 8, 4096
    w = make_decoder_weights(shape, 0)
    k, v = make_kv(shape, 0, B, ctx, 0)
    tokens = np.arange(B, dtype=np.int32) * 977 % shape.vocab
    pos = np.full(B, ctx - 1, np.int32)
    moe_s = [0.0]

    def moe_fn(l, xn):
        t0 = time.perf_counter()
        out = oracle.moe_forward(np.ascontiguousarray(xn), w.moe[l])[0]
        moe_s[0] += time.perf_counter() - t0
        return out
    t0 = time.perf_counter()
    r = dor.decoder_step(w, [k], [v], tokens, pos, moe_fn)
    t_all = time.perf_counter() - t0
    t0 = time.perf_counter()
    dor.linear(r["xn"], w.unembed)
    t_head = time.perf_counter() - t0
    t_layer = t_all - t_head
    t_step = full.n_layers * t_layer + t_head * full.vocab / vocab_slice
    desc = (f"one decode step of batch {B}: 1 of {full.n_layers} layers at the real widths ({t_layer:.2f} s, of which "
            f"MoE {moe_s[0]:.2f} s) and {vocab_slice} of {full.vocab} unembedding rows ({t_head:.2f} s), "
            f"extrapolated to the whole step ({t_step:.1f} s); numpy float64 + OpenMP C MoE")
    return B / t_step, oracle.n_threads(), desc


def water_oracle_params(cfg):
    from oracle import water
    nx, ny, nz = cfg.grid_dim
    p = water.WaterParams(cfg.n_particles, nx, ny, nz, cfg.cell_size, cfg.over_relaxation, cfg.rest_density, cfg.damping,
                          cfg.mass, cfg.dt)
    p.box_min[:] = cfg.box_min
    p.box_max[:] = cfg.box_max
    p.gravity[:] = cfg.gravity
    p.collision_substeps, p.jacobi_iterations = cfg.collision_substeps, cfg.jacobi_iterations
    return p


def water_cpu_steps(n_steps):
    """Times n_steps of the water step on one host core: the reference shader compiled for the CPU
    when that library is present, else the restatement.  Returns (steps/s, kind, description)."""
    from oracle import water
    from neonengine_b200.water_synth import WaterConfig, spawn_particles
    cfg = WaterConfig()
    pos, vel = spawn_particles(cfg), None
    vel = np.zeros_like(pos)
    prm = water_oracle_params(cfg)
    if water.have_ref():
        kind, fn, what = "reference", water.ref_step, "water_grid.comp compiled for the CPU, invocations run serially"
    else:
        kind, fn, what = "port", lambda p, a, b, n: water.step(p, a, b, n, collision_mode=0), "C restatement of water_grid.comp"
        water.lib()
    t0 = time.perf_counter()
    fn(prm, pos, vel, n_steps)
    dt = time.perf_counter() - t0
    return n_steps / dt, kind, f"{n_steps} steps of the same workload from the same start ({what}, 1 thread, {dt:.1f} s)"


def run_water_reference(args):
    n = max(1, min(args.steps, 20))
    sps, kind, desc = water_cpu_steps(n)
    line = {"impl": "reference", "metric": "water_steps_per_s", "value": sps, "unit": "steps/s", "n_gpus": args.gpus,
            "steps": n, "warmup": 0, "ms_per_step": 1e3 / sps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "water", "description": WORKLOADS["water"][3]},
            "cpu_baseline": {"value": sps, "unit": "steps/s", "cores": 1, "kind": kind, "sample": desc},
            "e2e": {"value": sps, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def run_water(args, local_rank):
    """The water step does not shard: N independent replicas under torchrun."""
    import torch
    import torch.distributed as dist
    from neonengine_b200.water_physics import WaterPhysics
    from neonengine_b200.water_synth import WaterConfig, spawn_particles
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = WaterConfig()
    pos0 = spawn_particles(cfg)
    sim = WaterPhysics(cfg, pos0, device=local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    st = torch.cuda.current_stream()
    warm = max(args.warmup, 3)
    sim.run_simulation(warm, stream=st)
    barrier()
    l0 = sim.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        sim.run_simulation(args.steps, stream=st)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        launches = sim.launch_count() - l0
        prof = [sim.profile_step() for _ in range(5)][1:]
        groups = {k: sum(p[k] for p in prof) / len(prof) for k in prof[0]}
        # end to end: host particle arrays in and out every step
        e2e_steps = max(10, min(args.steps, 200))
        pos_pin = torch.from_numpy(pos0.copy()).pin_memory()
        vel_pin = torch.zeros_like(pos_pin).pin_memory()
        for _ in range(3):
            sim.run_host_ptr(pos_pin.data_ptr(), vel_pin.data_ptr(), 1)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            sim.run_host_ptr(pos_pin.data_ptr(), vel_pin.data_ptr(), 1)
        e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    peaks, peak_kind = measured_peaks()
    C, N = cfg.n_cells, cfg.n_particles
    # dominant group: the 50 Jacobi launches; each reads flags, s, u, v, w, density, p and writes p once per cell
    jac_bytes = C * 32
    jac_ms = groups["jacobi"] / max(cfg.jacobi_iterations, 1)
    achieved = jac_bytes / (jac_ms * 1e-3) / 1e9
    line = {"metric": "water_steps_per_s", "value": world * args.steps / (ms * 1e-3), "unit": "steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "water", "description": WORKLOADS["water"][3], "particles": N, "cells": C,
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (the step does not shard)",
                       "l2_policy": "the whole state (5 MB of grids, 0.25 MB of particles) is far below the 126 MB L2 by "
                                    "the workload's own size; steps advance the simulation, no input repeats"},
            "e2e": {"value": world * e2e_steps / e2e_s, "unit": "steps/s", "h2d_bytes_per_step": 2 * N * 16,
                    "d2h_bytes_per_step": 2 * N * 16, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "k_jacobi (one of 50 launches per step; L2-resident 5 MB working set)",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "algorithmic_bytes_per_launch": jac_bytes,
                         "ms_per_launch": jac_ms, "eager_group_ms_per_step": groups,
                         "note": "launch-latency bound: 64 kernels per step over a working set that fits L2"},
            "clocks": clocks.summary()}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sps, kind, desc = water_cpu_steps(20)
        line["cpu_baseline"] = {"value": sps, "unit": "steps/s", "cores": 1, "kind": kind, "sample": desc}
    if rank == 0:
        emit(line)
    sim.close()
    if world > 1:
        dist.destroy_process_group()


SVGF_W, SVGF_H, SVGF_ITERS, SVGF_FRAMES = 1920, 1080, 3, 4


def svgf_cpu_frames(n_frames, w=SVGF_W, h=SVGF_H):
    """Times n_frames of the denoiser on one host core: the reference shaders compiled for the CPU
    when that library is present, else the restatement.  Returns (frames/s, kind, description)."""
    from neonengine_b200 import svgf_synth
    from oracle import svgf
    st = svgf.State.zeros(w, h)
    frames = [svgf_synth.make_frame(w, h, i) for i in range(n_frames)]
    if svgf.have_ref():
        kind, fn, what = "reference", svgf.ref_frame, "raytracing_pp.comp + raytracing_atrous.comp compiled for the CPU, bodies live"
        svgf.ref_lib()
    else:
        kind, fn, what = "port", lambda g, im, s, it: svgf.frame(g, im, s, it, serial=True), "C restatement of the two shaders"
        svgf.lib()
    t0 = time.perf_counter()
    for g, image in frames:
        fn(g, image, st, SVGF_ITERS)
    dt = time.perf_counter() - t0
    return n_frames / dt, kind, f"{n_frames} frames of the same {w}x{h} sequence ({what}, 1 thread, {dt:.1f} s)"


def run_svgf_reference(args):
    n = max(1, min(args.steps, 4))
    fps, kind, desc = svgf_cpu_frames(n)
    line = {"impl": "reference", "metric": "denoised_frames_per_s", "value": fps, "unit": "frames/s", "n_gpus": args.gpus,
            "steps": n, "warmup": 0, "ms_per_step": 1e3 / fps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "svgf", "description": WORKLOADS["svgf"][3]},
            "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": 1, "kind": kind, "sample": desc},
            "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def run_svgf(args, local_rank):
    """Frames are independent jobs per GPU (the history couples consecutive frames of one view):
    N independent replicas under torchrun."""
    import torch
    import torch.distributed as dist
    from neonengine_b200 import svgf_synth
    from neonengine_b200.svgf_denoiser import SvgfDenoiser
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w, h = SVGF_W, SVGF_H
    px = w * h
    dn = SvgfDenoiser(w, h, SVGF_ITERS, device=local_rank)
    frames = [svgf_synth.make_frame(w, h, i) for i in range(SVGF_FRAMES)]
    d_g = [[torch.from_numpy(a).cuda() for a in g] for g, _ in frames]
    d_img = [torch.from_numpy(im).cuda() for _, im in frames]
    d_work = [torch.empty_like(t) for t in d_img]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    st = torch.cuda.current_stream()

    def step(i):
        k = i % SVGF_FRAMES
        dn.render(d_g[k], d_work[k], stream=st)

    for k in range(SVGF_FRAMES):
        d_work[k].copy_(d_img[k])
    warm = max(args.warmup, 3, 2 * SVGF_FRAMES)   # every (frame, ping-pong parity) pair has its graph before timing
    for i in range(warm):
        step(i)
    barrier()
    l0 = dn.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for i in range(args.steps):
            step(i)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        launches = dn.launch_count() - l0
        prof = [dn.profile_frame(d_g[i % SVGF_FRAMES], d_work[i % SVGF_FRAMES], stream=st) for i in range(6)][2:]
        t_ms = sum(p[0] for p in prof) / len(prof)
        a_ms = sum(p[1] for p in prof) / len(prof)
        # end to end: the five host images of a frame in, the denoised image out, every frame
        e2e_steps = max(4, min(args.steps, 40))
        pin_g = [[torch.from_numpy(a).pin_memory() for a in g] for g, _ in frames]
        pin_img = [torch.from_numpy(im.copy()).pin_memory() for _, im in frames]
        for i in range(2):
            dn.render_host_ptr(*(t.data_ptr() for t in pin_g[i % SVGF_FRAMES]), pin_img[i % SVGF_FRAMES].data_ptr(), stream=st)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            dn.render_host_ptr(*(t.data_ptr() for t in pin_g[i % SVGF_FRAMES]), pin_img[i % SVGF_FRAMES].data_ptr(), stream=st)
        e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    peaks, peak_kind = measured_peaks()
    # one filter pass per pixel: reads normal 16 + position 16 + moments 16 + colour 8, writes image 4 + moments 16
    pass_bytes = px * 76
    pass_ms = a_ms / SVGF_ITERS
    achieved = pass_bytes / (pass_ms * 1e-3) / 1e9
    gbuf_mb = SVGF_FRAMES * px * 68 / 1e6
    line = {"metric": "denoised_frames_per_s", "value": world * args.steps / (ms * 1e-3), "unit": "frames/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "svgf", "description": WORKLOADS["svgf"][3], "width": w, "height": h,
                       "atrous_iterations": SVGF_ITERS,
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (one view per GPU)",
                       "l2_policy": f"{SVGF_FRAMES} rotating frames; their {gbuf_mb:.0f} MB of G-buffer and image exceed the 126 MB L2"},
            "e2e": {"value": world * e2e_steps / e2e_s, "unit": "frames/s", "h2d_bytes_per_step": px * 68,
                    "d2h_bytes_per_step": px * 4, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "k_atrous (one of 3 launches per frame)", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "traffic": None, "algorithmic_bytes_per_launch": pass_bytes, "ms_per_launch": pass_ms,
                         "eager_group_ms_per_frame": {"temporal": t_ms, "atrous": a_ms},
                         "note": "25 taps x ~80 unfused float operations per pixel: bound by the FP32 pipe, not by HBM"},
            "clocks": clocks.summary()}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        fps, kind, desc = svgf_cpu_frames(3)
        line["cpu_baseline"] = {"value": fps, "unit": "frames/s", "cores": 1, "kind": kind, "sample": desc}
    if rank == 0:
        emit(line)
    dn.close()
    if world > 1:
        dist.destroy_process_group()


PT_W, PT_H = 800, 600


def pt_cpu_frames(n_frames):
    """Times n_frames of the path tracer on one host core: the reference shaders compiled for the CPU when
    that library is present, else the restatement.  Returns (Mrays/s, kind, description)."""
    from neonengine_b200 import pt_synth
    from oracle import pt
    sc = pt_synth.cornell_box(0)
    ip, iv = pt_synth.camera(PT_W, PT_H)
    if pt.have_ref():
        kind, fn, what = "reference", pt.ref_render, "raygen.rgen + closesthit.rchit + miss shaders compiled for the CPU"
    else:
        kind, fn, what = "port", pt.render, "C restatement of the four shaders"
    rays, t0 = 0, time.perf_counter()
    for i in range(n_frames):
        rays += fn(sc, ip, iv, float(i), PT_W, PT_H)[1]
    dt = time.perf_counter() - t0
    return rays / dt / 1e6, kind, f"{n_frames} frames of the same scene and camera ({what}, own CPU hierarchy, 1 thread, {dt:.1f} s)"


def run_pt_reference(args):
    n = max(1, min(args.steps, 3))
    mr, kind, desc = pt_cpu_frames(n)
    line = {"impl": "reference", "metric": "path_tracer_mrays_per_s", "value": mr, "unit": "Mrays/s", "n_gpus": args.gpus,
            "steps": n, "warmup": 0, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": "pt", "description": WORKLOADS["pt"][3]},
            "cpu_baseline": {"value": mr, "unit": "Mrays/s", "cores": 1, "kind": kind, "sample": desc},
            "e2e": {"value": mr, "unit": "Mrays/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def run_pt(args, local_rank):
    """Frames are independent: N independent replicas under torchrun (one view per GPU)."""
    import torch
    import torch.distributed as dist
    from neonengine_b200 import pt_synth
    from neonengine_b200.path_tracer import PathTracer
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sc = pt_synth.cornell_box(0)
    ip, iv = pt_synth.camera(PT_W, PT_H)
    tr = PathTracer(sc, PT_W, PT_H, device=local_rank)
    img = torch.empty((PT_H, PT_W, 4), dtype=torch.uint8, device=f"cuda:{local_rank}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    st = torch.cuda.current_stream()
    warm = max(args.warmup, 3)
    for i in range(warm):
        tr.render(ip, iv, float(i), image=img, stream=st)
    barrier()
    tr.rays()
    l0 = tr.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for i in range(args.steps):
            tr.render(ip, iv, float(100 + i), image=img, stream=st)   # a new sample of the scene every frame
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        rays = tr.rays()
        launches = tr.launch_count() - l0
        e2e_steps = max(5, min(args.steps, 200))
        h_img = torch.empty((PT_H, PT_W, 4), dtype=torch.uint8).pin_memory()
        for i in range(3):
            tr.render_host_ptr(ip, iv, float(i), h_img.data_ptr())
        barrier()
        tr.rays()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            tr.render_host_ptr(ip, iv, float(500 + i), h_img.data_ptr())
        e2e_s = time.perf_counter() - t0
        e2e_rays = tr.rays()
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    peaks, peak_kind = measured_peaks()
    nodes, depth = tr.bvh_info()
    # algorithmic bytes of a frame: the rgba8 image out; the scene (0.9 MB of hierarchy, triangles, vertices) stays in L2
    frame_bytes = PT_W * PT_H * 4
    achieved = frame_bytes / (ms / args.steps * 1e-3) / 1e9
    line = {"metric": "path_tracer_mrays_per_s", "value": world * rays / (ms * 1e-3) / 1e6, "unit": "Mrays/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "pt", "description": WORKLOADS["pt"][3], "width": PT_W, "height": PT_H,
                       "rays_per_frame": rays / max(args.steps, 1), "bvh_nodes": nodes, "bvh_depth": depth,
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (one view per GPU)",
                       "l2_policy": "the scene (under 1 MB) is L2-resident by the workload's own size; every frame is a new sample "
                                    "(new frame id), nothing repeats"},
            "e2e": {"value": world * e2e_rays / e2e_s / 1e6, "unit": "Mrays/s", "h2d_bytes_per_step": 2 * 64 + 4,
                    "d2h_bytes_per_step": frame_bytes, "steps": e2e_steps, "frames_per_s": world * e2e_steps / e2e_s},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "pt_frame_kernel (one launch per frame)", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                         "algorithmic_bytes_per_launch": frame_bytes, "ms_per_launch": ms / args.steps,
                         "note": "latency- and divergence-bound traversal over an L2-resident scene: the HBM roofline does not bind; "
                                 "Mrays/s is the figure of merit"},
            "clocks": clocks.summary()}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        mr, kind, desc = pt_cpu_frames(2)
        line["cpu_baseline"] = {"value": mr, "unit": "Mrays/s", "cores": 1, "kind": kind, "sample": desc}
    if rank == 0:
        emit(line)
    tr.close()
    if world > 1:
        dist.destroy_process_group()


def run_decoder_reference(args):
    tps, cores, desc = decoder_cpu_sample()
    line = {"impl": "reference", "metric": "decoder_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": 1, "warmup": 0, "ms_per_step": 8 / tps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "cfg3", "description": WORKLOADS["cfg3"][3]},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def run_decoder(args, local_rank):
    """cfg3: N independent replicas of the decoder (one per GPU; the stack does not shard),
    value = tokens all replicas produce per second."""
    import torch
    import torch.distributed as dist
    from neonengine_b200.decoder_synth import AttentionWeights, DecoderShape
    from neonengine_b200.decoder_system import DecoderSystem
    from neonengine_b200.synth import MoeWeights

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", local_rank)
    shape = DecoderShape()
    if args.decoder_layers:
        shape.n_layers = args.decoder_layers
    B, ctx = 8, 4096
    H = shape.hidden
    dec = DecoderSystem(shape, B, ctx, device=local_rank)
    for opt in args.option:
        name, value = opt.split("=")
        dec.set_option(name, int(value))
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)

    def normal(dims, std, mean=0.0):
        return (torch.randn(dims, generator=gen, device=dev, dtype=torch.float32) * std + mean).to(torch.bfloat16).contiguous()

    embed, unembed = normal((shape.vocab, H), 0.02), normal((shape.vocab, H), 0.02)
    dec.set_embeddings(embed, unembed, normal((H,), 0.1, 1.0))
    del embed, unembed
    # expert tensors: one seeded host generation, uploaded once; every layer keeps its own
    # re-tiled copy in HBM (distinct memory), routers and attention blocks differ per layer
    mw = synth.make_weights(shape.moe, 0)
    dev_moe = [torch.from_numpy(a).to(dev) for a in (mw.gate_up_blocks, mw.gate_up_scales, mw.gate_up_bias.view(np.int16),
                                                     mw.down_blocks, mw.down_scales, mw.down_bias.view(np.int16))]
    for l in range(shape.n_layers):
        dec.set_attention(l, AttentionWeights(
            ln1=normal((H,), 0.1, 1.0), wqkv=normal((shape.qkv_rows, H), 0.02), bqkv=normal((shape.qkv_rows,), 0.02),
            sinks=normal((shape.n_q_heads,), 1.0), wo=normal((H, shape.q_dim), 0.02), bo=normal((H,), 0.02),
            ln2=normal((H,), 0.1, 1.0)))
        dec.set_moe(l, MoeWeights(shape.moe, normal((shape.moe.n_experts, H), 0.02), normal((shape.moe.n_experts,), 0.02),
                                  dev_moe[0], dev_moe[1], dev_moe[2], dev_moe[3], dev_moe[4], dev_moe[5]))
        dec.load_kv(l, normal((B, ctx - 1, shape.n_kv_heads, 64), 1.0), normal((B, ctx - 1, shape.n_kv_heads, 64), 1.0))
    del dev_moe
    torch.cuda.synchronize()

    tokens = (torch.arange(B, device=dev, dtype=torch.int32) * 977 + 11 * rank) % shape.vocab
    positions = torch.full((B,), ctx - 1, device=dev, dtype=torch.int32)
    pos_host = np.full(B, ctx - 1, np.int32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(n):  # the argmax of one step is the next step's input token
        for _ in range(n):
            dec.step(tokens, positions, next_tokens=tokens)

    warm = max(args.warmup, 3)
    run(warm)
    barrier()
    l0 = dec.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        run(args.steps)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        launches = dec.launch_count() - l0
        dense_b, kv_b, moe_b = dec.step_bytes(pos_host)
        # end to end: host token ids in, host next tokens out, one blocking call per step
        e2e_steps = max(10, min(args.steps, 200))
        tok_pin = torch.from_numpy(tokens.cpu().numpy().copy()).pin_memory()
        pos_pin = torch.from_numpy(pos_host.copy()).pin_memory()
        nxt_pin = torch.zeros(B, dtype=torch.int32).pin_memory()
        for _ in range(3):
            dec.step_host_ptr(tok_pin.data_ptr(), pos_pin.data_ptr(), B, nxt_pin.data_ptr())
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            dec.step_host_ptr(tok_pin.data_ptr(), pos_pin.data_ptr(), B, nxt_pin.data_ptr())
            tok_pin.copy_(nxt_pin)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([ms, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    step_s = ms / args.steps * 1e-3
    peaks, peak_kind = measured_peaks()
    step_bytes = dense_b + kv_b + moe_b
    achieved = step_bytes / step_s / 1e9
    line = {"metric": "decoder_tokens_per_s", "value": world * B / step_s, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg3", "description": WORKLOADS["cfg3"][3], "batch": B, "cache_tokens": ctx,
                       "layers": shape.n_layers,
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (the stack does not shard)",
                       "l2_policy": f"each step streams {step_bytes / 1e9:.1f} GB of weights and cache, far beyond the 126 MB L2; "
                                    "the tokens of a step are the previous step's argmax"},
            "e2e": {"value": world * B * e2e_steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * 4,
                    "d2h_bytes_per_step": B * 4, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "whole decode step (one CUDA graph of %d kernels)" % (launches // max(args.steps, 1)),
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "algorithmic_bytes_per_launch": step_bytes,
                         "bytes": {"dense_weights": dense_b, "kv_cache": kv_b, "moe_experts_touched": moe_b},
                         "ms_per_launch": ms / args.steps},
            "clocks": clocks.summary()}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, cores, desc = decoder_cpu_sample()
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}
    if rank == 0:
        emit(line)
    dec.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side-configs", action="store_true",
                    help="default run only: skip the cfg0 and cfg2 blocks measured beside the headline workload")
    ap.add_argument("--ep-nccl-exchange", action="store_true",
                    help="multi-GPU runs only: exchange rows with grouped ncclSend/ncclRecv instead of the library's own peer stores")
    ap.add_argument("--no-n1-base", action="store_true",
                    help="multi-GPU runs only: skip rank 0's single-GPU run of the same workload")
    ap.add_argument("--decoder-layers", type=int, default=None,
                    help="cfg3 only: run fewer than 24 layers (for small profiler captures; not a bench result)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library option to set before timing (e.g. pdl=0); for experiments")
    args = ap.parse_args()
    claim_stdout()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload is None:
        args.workload = "cfg1" if max(world, args.gpus) == 1 else "cfg4"
    if args.steps is None:
        args.steps = 200 if args.workload == "cfg3" else 500 if args.workload == "water" else 200 if args.workload in ("svgf", "pt") else 2000 if WORKLOADS[args.workload][0] <= 64 else 50
    if args.impl == "reference":
        if args.workload == "cfg3":
            if rank == 0:
                run_decoder_reference(args)
            return
        if args.workload == "water":
            if rank == 0:
                run_water_reference(args)
            return
        if args.workload == "svgf":
            if rank == 0:
                run_svgf_reference(args)
            return
        if args.workload == "pt":
            if rank == 0:
                run_pt_reference(args)
            return
        if args.steps > 64:
            args.steps = 8
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from neonengine_b200.moe_layer_system import MoeLayerSystem

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU: the MoE layer has no CPU path")
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    if args.workload == "cfg3":
        run_decoder(args, local_rank)
        return
    if args.workload == "water":
        run_water(args, local_rank)
        return
    if args.workload == "svgf":
        run_svgf(args, local_rank)
        return
    if args.workload == "pt":
        run_pt(args, local_rank)
        return

    run_moe(args, rank, world, local_rank)


def dram_traffic_table():
    """Measured DRAM bytes per launch (ncu captures) of the dominant kernels: lines
    `kernel workload bytes units commit` in profiles/dram_traffic.txt."""
    table = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if os.path.exists(path):
        for ln in open(path):
            f = ln.split()
            if len(f) >= 5 and not ln.startswith("#"):
                table[(f[0], f[1])] = {"bytes": float(f[2]), "units": float(f[3]), "commit": f[4]}
    return table


def disjoint_decode_batches(W, n_batches, base_stream=0):
    """Single-token batches whose expert sets are pairwise disjoint where the draw allows it, so that
    n_batches * top_k distinct experts (all 32 at the default shape) rotate through the timed region
    and no pass finds its weights in L2."""
    k = W.shape.top_k
    picked, used = [], set()
    for stream in range(base_stream, base_stream + 4000):
        hid = synth.make_hidden(1, W, 0, stream=stream)
        lg = synth.router_logits_f64(hid, W)[0]
        top = set(np.argsort(-lg)[:k].tolist())
        if not (top & used):
            picked.append(hid)
            used |= top
            if len(picked) == n_batches:
                return picked
        if len(used) + k > W.shape.n_experts:
            used = set()   # every expert has been used once: start another round
    while len(picked) < n_batches:
        picked.append(synth.make_hidden(1, W, 0, stream=base_stream + 5000 + len(picked)))
    return picked


def parity_sample(hidden, lb, got_out, got_idx, expert_weights, shape, sample):
    """Routing of every token and outputs of the sampled tokens against the CPU oracle.
    expert_weights(lo, hi) returns the MoeWeights of experts [lo, hi) (full router)."""
    import oracle
    router = expert_weights(0, 1)
    ridx, rw = oracle.route(hidden, router.router_w, router.router_b, shape.top_k, lb)
    mism = int((ridx != got_idx).any(axis=1).sum())
    sample = np.asarray(sample, np.int32)
    ref = np.zeros((sample.size, shape.hidden), np.float64)
    for e in sorted(set(ridx[sample].ravel().tolist())):
        ref += oracle.experts(hidden, ridx, rw, expert_weights(e, e + 1), tokens=sample, e_lo=e)
    got = np.asarray(got_out, np.float64)[sample]
    max_abs = float(np.abs(got - ref).max())
    mean_rel = float(np.abs(got - ref).mean() / max(np.abs(ref).mean(), 1e-30))
    return {"routing_mismatches": mism, "tokens_routed": int(hidden.shape[0]), "tokens": int(sample.size),
            "max_abs": max_abs, "mean_rel": mean_rel,
            "pass": bool(mism == 0 and max_abs <= 2e-2 and mean_rel <= 5e-3),
            "oracle": "CPU restatement of the configuration text, fp64 accumulate (parity unpinned: the reference has no such path)"}


class MoeRun:
    """One workload on one layer: device-timed groups of K steps, per-stage profile, roofline, parity."""

    def __init__(self, workload, args, rank, world, local_rank, dist, weights=None, min_seconds=0.3):
        import torch
        from neonengine_b200.moe_layer_system import MoeLayerSystem
        self.torch, self.dist, self.args = torch, dist, args
        self.workload, self.rank, self.world, self.local_rank = workload, rank, world, local_rank
        self.T, self.E, self.zipf, self.desc = WORKLOADS[workload]
        self.shape = synth.MoeShape(n_experts=self.E)
        self.ep = world > 1
        self.nl = self.E // world
        self.min_seconds = min_seconds
        if weights is not None:
            self.W = weights
        else:
            self.W = synth.make_weights(self.shape, 0, experts=(rank * self.nl, (rank + 1) * self.nl) if self.ep else None)
        T = self.T
        self.decode = T <= 64
        self.n_batches = 8 if self.decode else 2
        if T == 1 and not self.ep:
            self.batches, self.lb = disjoint_decode_batches(self.W, self.n_batches), None
        else:
            self.batches, self.lb = make_batches(T, self.W, self.zipf, self.n_batches, base_stream=100 * rank)
        self.dev = torch.device("cuda", local_rank)
        self.layer = MoeLayerSystem(self.shape, self.W, max_tokens=T, device=local_rank, ep_rank=rank if self.ep else 0,
                                    ep_size=world if self.ep else 1)
        for opt in args.option:
            name, value = opt.split("=")
            self.layer.set_option(name, int(value))
        self.d_batches = [torch.from_numpy(b.view(np.int16)).to(self.dev) for b in self.batches]
        self.d_lb = None if self.lb is None else torch.from_numpy(self.lb).to(self.dev)
        self.d_out = torch.empty((T, self.shape.hidden), dtype=torch.float32, device=self.dev)
        self.run = self.layer.run_ep if self.ep else self.layer.run

    def barrier(self):
        if self.ep:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.ep:
            t = self.torch.tensor([v], device=self.dev, dtype=self.torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return v

    def step_device(self, i):
        self.run(self.d_batches[i % self.n_batches], logit_bias=self.d_lb, out=self.d_out)

    def timed(self, fn, steps):
        torch = self.torch
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        ev0.record()
        for i in range(steps):
            fn(i)
        ev1.record()
        self.barrier()
        return self.max_over_ranks(ev0.elapsed_time(ev1))

    def warm(self, warmup):
        # the library captures a pass into a CUDA graph the second time it sees the same arguments, so
        # every rotating batch goes through twice before the warm-up proper
        for i in range(2 * self.n_batches):
            self.step_device(i)
        for i in range(max(warmup, 3)):
            self.step_device(i)

    def timed_groups(self, steps):
        """Groups of exactly `steps` steps, repeated until min_seconds of timed work have run (the
        elapsed time is the maximum over ranks, so every rank runs the same number of groups)."""
        groups, total = [], 0.0
        while True:
            ms = self.timed(self.step_device, steps)
            groups.append(ms)
            total += ms
            if total >= self.min_seconds * 1e3 or len(groups) >= 400:
                return groups

    def stage_profile(self, steps):
        layer = self.layer
        if self.ep:
            acc, rows, n = {}, 0, 0
            for i in range(min(steps, 20)):
                self.step_device(i)
                tms, r = layer.ep_times()
                rows += r
                for kk, v in tms.items():
                    acc[kk] = acc.get(kk, 0.0) + v
                n += 1
            return {kk: self.max_over_ranks(v / n) for kk, v in acc.items()}, rows / n
        layer.profile(True)
        self.timed(self.step_device, min(max(steps, 50), 2000))
        stage_ms, n = layer.read_profile()
        layer.profile(False)
        return {kk: v / max(n, 1) for kk, v in stage_ms.items()}, n

    def touched(self):
        counts = []
        for bt in self.d_batches:
            self.layer.run(bt, logit_bias=self.d_lb, out=self.d_out)
            counts.append(int((self.layer.read_dispatch()[0] > 0).sum()))
        return sum(counts) / len(counts)

    def parity(self, n_sample):
        torch = self.torch
        T = self.T
        hid = self.batches[0]
        out, idx, _ = self.run(self.d_batches[0], logit_bias=self.d_lb, want_routing=True)
        torch.cuda.synchronize()
        sample = np.unique(np.linspace(0, T - 1, min(T, n_sample)).astype(np.int32))
        if self.ep:
            def weights(lo, hi):
                return synth.make_weights(self.shape, 0, experts=(lo, hi))
        else:
            def weights(lo, hi):
                return self.W.slice_experts(lo, hi)
        return parity_sample(hid, self.lb, out.cpu().numpy(), idx.cpu().numpy(), weights, self.shape, sample)

    def mxf4_variant(self, steps, ceil4):
        """The same workload with option mxf4_prefill: activations quantised to MXFP4, both expert products on
        tcgen05.mma.kind::mxf4.  Outside the accuracy contract by construction (4-bit activations), so it is
        reported beside the default path, with its error against the quantisation-aware oracle and the plain one."""
        import oracle
        torch, shape, T, k = self.torch, self.shape, self.T, self.shape.top_k
        self.layer.set_option("mxf4_prefill", 1)
        try:
            self.warm(3)
            groups = self.timed_groups(steps)
            ms = statistics.median(groups) / steps
            stage_ms, _ = self.stage_profile(steps)
            out, idx, _ = self.run(self.d_batches[0], logit_bias=self.d_lb, want_routing=True)
            torch.cuda.synchronize()
            hid = self.batches[0]
            ridx, rw = oracle.route(hid, self.W.router_w, self.W.router_b, k, self.lb)
            sample = np.unique(np.linspace(0, T - 1, 6).astype(np.int32))
            got = out.cpu().numpy().astype(np.float64)[sample]
            ref_q = oracle.experts(hid, ridx, rw, self.W, tokens=sample, quant_act=True)
            ref = oracle.experts(hid, ridx, rw, self.W, tokens=sample)
            eq = np.abs(got - ref_q)
            layer_tf = T * k * shape.flops_per_pair / (ms * 1e-3) / 1e12
            gemm_tf = T * k * shape.flops_per_pair / ((stage_ms["gate_up"] + stage_ms["down"]) * 1e-3) / 1e12
            return {"option": "mxf4_prefill=1 (MXFP4-quantised activations, tcgen05.mma.kind::mxf4.block_scale.scale_vec::2X)",
                    "ms_per_step": ms, "value": T / (ms * 1e-3), "unit": "tokens/s", "stage_ms_per_step": stage_ms,
                    "layer_tflops": layer_tf, "layer_frac_of_mxf4_ceiling": layer_tf / ceil4,
                    "layer_frac_of_mxfp4_nominal_9000": layer_tf / 9000.0,
                    "expert_gemms_tflops": gemm_tf, "expert_gemms_frac_of_mxf4_ceiling": gemm_tf / ceil4,
                    "expert_gemms_frac_of_mxfp4_nominal_9000": gemm_tf / 9000.0,
                    "parity_vs_quantisation_aware_oracle": {
                        "routing_mismatches": int((ridx != idx.cpu().numpy()).any(axis=1).sum()), "tokens": int(sample.size),
                        "max_abs": float(eq.max()), "mean_rel": float(eq.mean() / np.abs(ref_q).mean()),
                        "outputs_over_2e-2": float((eq > 2e-2).mean())},
                    "error_vs_plain_oracle": {"max_abs": float(np.abs(got - ref).max()),
                                              "mean_rel": float(np.abs(got - ref).mean() / np.abs(ref).mean()),
                                              "note": "4-bit activations: outside the 2e-2 / 5e-3 contract by construction"}}
        finally:
            self.layer.set_option("mxf4_prefill", 0)

    def close(self):
        self.layer.close()
        del self.d_batches, self.d_out


def moe_roofline(run, step_s, stage_ms, n_prof, peaks, peak_kind, traffic_table):
    """The dominant kernel's roofline for a single-GPU MoE workload."""
    shape, T, k = run.shape, run.T, run.shape.top_k
    H, I = shape.hidden, shape.inter
    mean_touched = run.touched()
    layer_bytes = mean_touched * shape.expert_bytes + shape.router_bytes + T * H * 2 + T * H * 4
    gu_expert_bytes = 2 * I * H // 2 + 2 * I * H // 32 + 2 * I * 2
    if run.layer.launch_count and T <= 8 and stage_ms is None:
        # one cooperative kernel per pass: the kernel is the layer, its algorithmic bytes are the layer's
        achieved = layer_bytes / step_s / 1e9
        roof = {"bound": "hbm", "kernel": "decode_fused_kernel (router + gate_up + SwiGLU + down + combine, one launch)",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None, "algorithmic_bytes_per_launch": layer_bytes,
                "ms_per_launch": step_s * 1e3,
                "note": "launch duration = the step (one kernel per pass, replayed from a CUDA graph; CUDA events around K passes)"}
    elif run.decode:
        gu_ms = stage_ms["gate_up"]
        gu_bytes = mean_touched * gu_expert_bytes + T * H * 2 + T * k * I * 4
        achieved = gu_bytes / (gu_ms * 1e-3) / 1e9
        # passes of up to 96 tokens run the grouped GEMM on CTA pairs (two-SM MMAs), larger ones on single CTAs
        kern = "gmm_pair_kernel" if run.layer.pair_ctas() > 0 else "gmm_bs_kernel"
        roof = {"bound": "hbm", "kernel": kern + "<gate_up>", "achieved": achieved, "peak": peaks["hbm_gbs"],
                "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                "algorithmic_bytes_per_launch": gu_bytes, "ms_per_launch": gu_ms}
        ent = traffic_table.get((kern + "_gate_up", run.workload))
        if ent:   # ncu capture of one launch, scaled by the experts this run touched
            roof["traffic"] = ent["bytes"] * mean_touched / ent["units"]
            roof["traffic_source"] = f"ncu capture at commit {ent['commit']} ({ent['bytes']:.0f} B at {ent['units']:.0f} experts touched), scaled"
    else:
        gu_ms = stage_ms["gate_up"]
        gu_flops = T * k * 2 * 2 * I * H
        achieved = gu_flops / (gu_ms * 1e-3) / 1e12
        peak = peaks.get("bf16_tflops", 1590.0)
        from neonengine_b200 import mma_rate
        ceil8 = mma_rate.measure("mxf8f6f4", 128, 8192, device=run.local_rank)["tflops"]
        ceil4 = mma_rate.measure("mxf4", 256, 8192, device=run.local_rank)["tflops"]
        layer_tf = T * k * shape.flops_per_pair / step_s / 1e12
        kern = "gmm_pair_prefill_kernel" if run.layer.pair_ctas() > 0 else "gmm_bs_kernel"
        roof = {"bound": "tensor", "kernel": kern + "<gate_up>", "achieved": achieved, "peak": peak,
                "peak_kind": peak_kind + " bf16 burst", "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                "algorithmic_flops_per_launch": gu_flops, "ms_per_launch": gu_ms, "layer_tflops": layer_tf,
                "layer_frac_of_mxfp4_nominal_9000": layer_tf / 9000.0,
                "mma_issue_ceiling_tflops": {"mxf8f6f4_128x128": ceil8, "mxf4_128x256": ceil4},
                "frac_of_mxf4_ceiling": achieved / ceil4, "layer_frac_of_mxf4_ceiling": layer_tf / ceil4}
    if stage_ms is not None:
        roof["stage_ms_per_step"] = stage_ms
    roof.update({"layer_bytes_per_step": layer_bytes, "layer_gbs": layer_bytes / step_s / 1e9,
                 "layer_frac_of_peak": layer_bytes / step_s / 1e9 / peaks["hbm_gbs"],
                 "layer_frac_of_8000": layer_bytes / step_s / 1e9 / 8000.0, "experts_touched_mean": mean_touched})
    return roof


def side_config(workload, args, local_rank, peaks, peak_kind, traffic_table):
    """A further configuration measured in the same run (its own layer, its own batches): device-timed
    ms/step, tokens/s, the dominant kernel's roofline and a parity sample."""
    run = MoeRun(workload, args, 0, 1, local_rank, None, min_seconds=0.15)
    run.warm(args.warmup)
    groups = run.timed_groups(args.steps)
    ms = statistics.median(groups)
    step_s = ms / args.steps * 1e-3
    fused = run.T <= 8 and not any(o.startswith("decode_fused=0") for o in args.option)
    stage_ms = None if fused else run.stage_profile(args.steps)[0]
    roof = moe_roofline(run, step_s, stage_ms, 0, peaks, peak_kind, traffic_table)
    out = {"description": run.desc, "tokens_per_step": run.T, "ms_per_step": ms / args.steps,
           "ms_per_step_min": min(groups) / args.steps, "groups": len(groups), "value": run.T / step_s, "unit": "tokens/s",
           "roofline": roof, "parity": run.parity(8), "status": run.layer.status()}
    if run.T > 224 and "mma_issue_ceiling_tflops" in roof:
        out["mxf4_variant"] = run.mxf4_variant(args.steps, roof["mma_issue_ceiling_tflops"]["mxf4_128x256"])
    run.close()
    return out


def run_moe(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    ep = world > 1
    peaks, peak_kind = measured_peaks()
    traffic_table = dram_traffic_table()
    T, E, zipf, desc = WORKLOADS[args.workload]
    if ep and E % world:
        raise SystemExit(f"{E} experts cannot be sharded over {world} ranks")

    # With several GPUs, rank 0 first runs the SAME workload on its GPU alone (all experts local, no
    # exchange): the like-for-like base of the weak-scaling numbers.
    n1_same = None
    if ep and not args.no_n1_base:
        if rank == 0:
            solo = MoeRun(args.workload, args, 0, 1, local_rank, None, min_seconds=0.1)
            solo.warm(3)
            g = solo.timed_groups(min(args.steps, 10))
            n1_same = statistics.median(g) / min(args.steps, 10)
            solo.close()
            del solo
            torch.cuda.empty_cache()
        dist.barrier()

    run = MoeRun(args.workload, args, rank, world, local_rank, dist)
    layer, shape = run.layer, run.shape
    H, I, k = shape.hidden, shape.inter, shape.top_k
    if ep:
        ids = [layer.ep_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        layer.ep_init(ids[0])

        def gather(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out
        ep_peer = (not args.ep_nccl_exchange) and layer.ep_enable_peer_stores(gather)
    n_batches, batches, lb = run.n_batches, run.batches, run.lb

    # pinned host buffers for the end-to-end arm
    h_in = [torch.from_numpy(b.view(np.int16)).pin_memory() for b in batches]
    h_out = torch.empty((T, H), dtype=torch.float32).pin_memory()
    h_outs = [torch.empty((T, H), dtype=torch.float32).pin_memory() for _ in range(4)]
    h_lb = None if lb is None else torch.from_numpy(lb).pin_memory()
    lbp = None if h_lb is None else h_lb.data_ptr()

    with ClockSampler(local_rank) as clocks:
        run.warm(args.warmup)
        l0 = layer.launch_count
        groups = run.timed_groups(args.steps)
        launches = (layer.launch_count - l0) // len(groups)
        ms = statistics.median(groups)
        fused = (not ep) and T <= 8 and not any(o.startswith("decode_fused=0") for o in args.option)
        stage_ms, ep_rows = (None, 0) if fused else run.stage_profile(args.steps)
        # end to end through host buffers: every step's hidden states come from pinned host memory and
        # its result goes back to pinned host memory inside the timed region
        e2e_steps = max(3, min(args.steps, 500))
        if not ep:
            for i in range(3):
                layer.run_host_ptr(h_in[i % n_batches].data_ptr(), T, lbp, h_out.data_ptr())
            run.barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                layer.run_host_ptr(h_in[i % n_batches].data_ptr(), T, lbp, h_out.data_ptr())
            run.barrier()
            e2e_blocking_s = time.perf_counter() - t0
        # the same steps through the pipelined call: upload of step i+1 and download of step i-1 overlap
        # the layer pass of step i (neon_moe_forward_host_batches; collective on an expert-parallel handle)
        ins = [h_in[i % n_batches].data_ptr() for i in range(e2e_steps)]
        outs = [h_outs[i % len(h_outs)].data_ptr() for i in range(e2e_steps)]
        layer.run_host_batches(ins[:4], T, lbp, outs[:4])
        run.barrier()
        t0 = time.perf_counter()
        layer.run_host_batches(ins, T, lbp, outs)
        run.barrier()
        e2e_s = run.max_over_ranks(time.perf_counter() - t0)
        if ep:
            e2e_blocking_s = e2e_s
    status = layer.status()
    assert status == 0, f"device status word {status}"

    tokens_per_step = T * world
    step_s = ms / args.steps * 1e-3
    value = tokens_per_step / step_s
    e2e_value = tokens_per_step * e2e_steps / e2e_s
    clk = clocks.summary()

    if ep:
        # dominant unit: the local expert pass (both grouped GEMMs) over the rows this rank received
        ep_ms = stage_ms
        ex_ms = ep_ms["experts"]
        achieved = ep_rows * shape.flops_per_pair / (ex_ms * 1e-3) / 1e12
        from neonengine_b200 import mma_rate
        ceil8 = mma_rate.measure("mxf8f6f4", 128, 8192, device=local_rank)["tflops"]
        ceil4 = mma_rate.measure("mxf4", 256, 8192, device=local_rank)["tflops"]
        roofline = {"bound": "tensor", "kernel": "gmm_bs_kernel (gate_up + down, local experts)", "achieved": achieved,
                    "peak": peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")), "peak_kind": peak_kind + " bf16 sustained",
                    "unit": "TFLOP/s", "traffic": None, "ms_per_launch": ex_ms,
                    "algorithmic_flops_per_launch": ep_rows * shape.flops_per_pair,
                    "ep_stage_ms_per_step_max_over_ranks": ep_ms, "rows_received_rank0": ep_rows,
                    "all_to_all_exposed_ms": ep_ms["dispatch_a2a"] + ep_ms["combine_a2a"],
                    "exchange": ("this library's own stores into the peers' buffers over NVLink (token rows by a scatter kernel, outputs from "
                                 "the down product's epilogue); NCCL gathers the histograms and orders the ranks"
                                 if ep_peer else "grouped ncclSend/ncclRecv"),
                    "mma_issue_ceiling_tflops": {"mxf8f6f4_128x128": ceil8, "mxf4_128x256": ceil4},
                    "frac_of_mxf4_ceiling": achieved / ceil4, "frac_of_mxfp4_nominal_9000": achieved / 9000.0}
        roofline["frac"] = achieved / roofline["peak"]
        if n1_same is None and rank == 0 and not args.no_n1_base:
            n1_same = None
        n1 = [n1_same if rank == 0 else None]
        dist.broadcast_object_list(n1, src=0)
        if n1[0] is not None:
            roofline["n1_same_workload_ms"] = n1[0]
            roofline["weak_efficiency_same_workload"] = n1[0] / (ms / args.steps)
    else:
        roofline = moe_roofline(run, step_s, stage_ms, 0, peaks, peak_kind, traffic_table)
    mxf4_variant = None
    if not ep and T > 224 and "mma_issue_ceiling_tflops" in roofline and not any(o.startswith("mxf4_prefill") for o in args.option):
        mxf4_variant = run.mxf4_variant(args.steps, roofline["mma_issue_ceiling_tflops"]["mxf4_128x256"])

    parity = run.parity(16 if ep else 8) if rank == 0 or ep else None
    if ep:   # the pass is collective: every rank ran it, rank 0 checked its own tokens
        parity = parity if rank == 0 else None

    weights_mb = shape.expert_bytes * run.nl / 1e6
    line = {"metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "tokens_per_step_per_gpu": T,
                       "hidden": H, "inter": I, "n_experts": E, "top_k": k,
                       "parallelism": "single GPU" if world == 1 else f"ep{world} (experts sharded, all-to-all over NCCL)",
                       "l2_policy": f"{n_batches} rotating batches; {weights_mb:.0f} MB of expert weights per GPU "
                                    "exceed the 126 MB L2"},
            "timing": {"groups_of_steps": len(groups), "ms_per_step_median": ms / args.steps,
                       "ms_per_step_min": min(groups) / args.steps, "ms_per_step_max": max(groups) / args.steps,
                       "timed_seconds": sum(groups) / 1e3,
                       "ms_per_step_x_sm_mhz": None if not clk["sm_mhz"] else ms / args.steps * clk["sm_mhz"]},
            "e2e": {"value": e2e_value, "unit": "tokens/s",
                    "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 4, "steps": e2e_steps,
                    "api": "neon_moe_forward_host_batches (pipelined copies" + ("; every batch an expert-parallel pass)" if ep else ")"),
                    "blocking_call_per_step_value": tokens_per_step * e2e_steps / e2e_blocking_s},
            "gpu_launches": int(launches), "roofline": roofline, "parity": parity, "clocks": clk}
    if mxf4_variant:
        line["mxf4_variant"] = mxf4_variant

    if rank == 0 and world == 1 and args.workload == "cfg1" and not args.no_side_configs:
        run.close()
        torch.cuda.empty_cache()
        line["configs"] = {w: side_config(w, args, local_rank, peaks, peak_kind, traffic_table) for w in ("cfg0", "cfg2")}
    if rank == 0 and not args.no_cpu_baseline:
        cpu_tps, cpu_steps_done, cores = cpu_steps(run.W if not ep else synth.make_weights(synth.MoeShape(n_experts=32), 0),
                                                   batches if not ep else make_batches(64, synth.make_weights(synth.MoeShape(n_experts=32), 0), False, 2)[0],
                                                   lb, seconds_budget=12.0 if not ep else 6.0, max_tokens_per_step=min(T, 64))
        line["cpu_baseline"] = {"value": cpu_tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"{cpu_steps_done} steps of {min(T, 64)} tokens "
                                          + ("of the same batches" if not ep else "of the 32-expert layer (the 128-expert weights of "
                                             "all ranks are not on one host; per-token work is the same)")
                                          + " (CPU oracle, OpenMP, fp64 accumulate)"}
    if rank == 0:
        emit(line)
    try:
        run.close()
    except Exception:
        pass
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
