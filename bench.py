#!/usr/bin/env python
"""Benchmark of the B200 Qwen4 MoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c0|c1|c2|c3|c4] [--impl reference]

A step is one pass of the MoE layer over one batch of synthetic tokens.  The default workload
(N = 1) is the 4-token decode / multi-token-verify batch with IQ2_XXS routed experts and a
Q4_K shared expert (hidden 2048, 512 experts, top-10, intermediate 512); the metric is
MoE-layer microseconds per token.  Successive steps run DIFFERENT layers (weight sets) in
rotation so that a step's weights are never in L2 from the previous pass over them.

One JSON line is printed by rank 0:
  value      device time (CUDA events around the K steps, activations resident in HBM)
  e2e        the same metric through qwen4_moe_forward with host buffers (H2D + D2H inside)
  roofline   the dominant kernel's algorithmic weight bytes / its event-timed duration
  layer      the whole layer's weight bytes touched / step time, against the HBM peak
  cpu_baseline  the reference's own CPU MoE path timed here on the host cores
`--impl reference` times only that CPU path and prints the same line shape.

With N > 1 (torchrun, one rank per GPU) the workload is the sharded one: batched decode of 64
sequences through 48 Q4_K layers with the 512 experts cut into N blocks (expert parallel), rows
exchanged by all-to-all over NCCL; `--workload c4` runs the same batch on one GPU for comparison.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from picoforge_b200 import abi, synth  # noqa: E402
from picoforge_b200.layer import MoeLayer  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised in profiles/ (ncu's replay adds cache write-backs to the write part; the read part equals
# the algorithmic bytes).
TRAFFIC = {
    "c1:fused_decode_kernel": 32.91e6 + 12.29e6,
    "c2:gate_up_routed": 144.26e6 + 17.5e6,
}

STAGES = ("router_logits", "route", "group", "gate_up_routed", "gate_up_shared", "down_routed", "down_shared", "combine")
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# ---- workloads ---------------------------------------------------------------------------------
def workload(name: str, layers: int):
    """Returns (description, tokens, [LayerSpec...], x)."""
    if name == "c1":
        specs = [synth.make_layer(1, layer=l, routed_type=abi.IQ2_XXS, shared_type=abi.Q4_K) for l in range(layers)]
        x = synth.activations(1, 4)
        synth.correlated_tokens(x, 1, 0, 1, 0.95)
        desc = "c1: 4-token decode, IQ2_XXS routed + Q4_K shared, 512 experts top-10, hidden 2048"
    elif name == "c0":
        specs = [synth.make_layer(0, layer=l, routed_type=abi.Q4_K, shared_type=abi.Q4_K) for l in range(layers)]
        x = synth.activations(0, 1)
        desc = "c0: 1-token decode, Q4_K, 512 experts top-10, hidden 2048"
    elif name == "c2":
        specs = []
        for l in range(layers):
            spec = synth.make_layer(0, layer=l, routed_type=abi.Q4_K, shared_type=abi.Q4_K)
            synth.zipf_router_bias(spec, 2 + l)
            specs.append(spec)
        x = synth.activations(2, 1024)
        x[:, 0] = 1.0
        desc = "c2: 1024-token prefill chunk, Q4_K, Zipf(1.1) expert popularity"
    elif name == "c3":
        specs = [synth.make_layer(3, layer=l, routed_type=abi.Q2_K, shared_type=abi.Q4_K) for l in range(layers)]
        x = synth.activations(3, 1024)
        desc = "c3 (one GPU): 1024-token prefill chunk, Q2_K routed + Q4_K shared, uniform routing"
    elif name == "c4":
        specs = []
        for l in range(layers):
            spec = synth.make_layer(4, layer=l, routed_type=abi.Q4_K, shared_type=abi.Q4_K)
            synth.zipf_router_bias(spec, 4 + l)
            specs.append(spec)
        x = synth.activations(4, 64)
        x[:, 0] = 1.0
        desc = "c4 (one GPU): batched decode, 64 sequences x 1 token, Q4_K, Zipf(1.1) expert popularity"
    else:
        raise SystemExit(f"unknown workload {name}")
    return desc, x.shape[0], specs, x


def stage_bytes(spec, ids):
    """Algorithmic weight bytes each kernel must read for this batch (distinct experts once)."""
    layouts = spec.layouts()
    distinct = len(np.unique(ids))
    per_expert = [l.expert_bytes for l in layouts]
    return {
        "router_logits": layouts[0].tensor_bytes + layouts[7].tensor_bytes,
        "route": 0, "group": 0,
        "gate_up_routed": distinct * (per_expert[1] + per_expert[2]),
        "gate_up_shared": layouts[4].tensor_bytes + layouts[5].tensor_bytes,
        "down_routed": distinct * per_expert[3], "down_shared": layouts[6].tensor_bytes, "combine": 0,
    }, distinct


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, device: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        n = self.nvml
        names = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.handle)
                self.reasons |= {name for name, bit in names.items() if mask & bit}
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nvml:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- CPU reference arm -------------------------------------------------------------------------
def cpu_reference_step(specs, x, repeats: int, warmup: int):
    """Times the reference's CPU MoE path (its own objects when built, else the oracle port)
    on one batch: tokens sharded over host threads, one workspace per thread."""
    import oracle
    cores = len(os.sched_getaffinity(0))
    tokens = x.shape[0]
    spec = specs[0]
    if oracle.reference_available():
        kind = "reference"
        api = oracle.reference_api()
        threads = max(1, min(cores, tokens))
        bounds = np.linspace(0, tokens, threads + 1).astype(int)
        layers = [MoeLayer(api, spec, int(bounds[i + 1] - bounds[i])) for i in range(threads)]   # created serially

        def run_once():
            workers = [threading.Thread(target=layers[i].forward, args=(x[bounds[i]:bounds[i + 1]], False))
                       for i in range(threads)]
            for w in workers:
                w.start()
            for w in workers:
                w.join()
    else:
        kind = "port"
        threads = max(1, min(cores, 64))

        def run_once():
            oracle.forward(spec, x, threads=threads)
    for _ in range(warmup):
        run_once()
    start = time.perf_counter()
    for _ in range(repeats):
        run_once()
    seconds = (time.perf_counter() - start) / repeats
    return seconds, threads, kind


# ---- main --------------------------------------------------------------------------------------
# ---- expert-parallel batched decode (C4) ------------------------------------------------------------
def run_expert_parallel(args, rank: int, local_rank: int, world: int) -> None:
    """64 concurrent sequences, one token each, through `--ep-layers` Q4_K layers with Zipf(1.1) expert
    popularity; the 512 experts are cut into `world` contiguous blocks, tokens are data-parallel, and
    rows travel to the experts' owners and back by all-to-all over NCCL (picoforge_b200/expert_parallel.py).
    Total work is fixed as N grows ("strong" scaling).  Time: CUDA events on the stream everything is
    enqueued on, maximum over ranks."""
    import torch
    import torch.distributed as dist
    from picoforge_b200.expert_parallel import EpLayer, TorchExchange

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    api = abi.product()
    lib = api.lib
    if lib.qw4cu_set_device(local_rank) != 0:
        raise SystemExit(lib.qw4cu_last_error().decode())
    lib.qw4cu_set_router_mode(1 if args.router == "fast" else 0)
    lib.qw4cu_set_tile_path(args.tile_path)
    tokens, n_layers = 64, args.ep_layers
    per, epr = tokens // world, 512 // world
    x_all = synth.activations(4, tokens)
    x_all[:, 0] = 1.0
    specs, layers = [], []
    for l in range(n_layers):
        spec = synth.make_layer(4, layer=l, routed_type=abi.Q4_K, shared_type=abi.Q4_K, shard=(rank * epr, epr))
        synth.zipf_router_bias(spec, 4 + l)
        specs.append(spec)
        layers.append(EpLayer(api, spec, per, world, rank, TorchExchange()))
        spec.tensors = []                                        # resident in HBM now: keep one layer of host bytes at a time
    stream = torch.cuda.Stream()
    pinned_x = torch.from_numpy(x_all[rank * per:(rank + 1) * per].copy()).pin_memory()
    pinned_y = torch.empty_like(pinned_x).pin_memory()
    with torch.cuda.stream(stream):
        x = pinned_x.cuda(non_blocking=True)

        def step():
            y = None
            for layer in layers:
                y = layer.forward(x)
            return y

        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        for layer in layers:
            layer.sync()
        dist.barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            before = lib.qw4cu_launch_count()
            begin.record(stream)
            for _ in range(args.steps):
                y = step()
            end.record(stream)
            stream.synchronize()
            launches = lib.qw4cu_launch_count() - before
        for layer in layers:
            layer.sync()                                                      # error words of every layer
        dist.barrier()
        elapsed = torch.tensor([begin.elapsed_time(end)], device="cuda")
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        ms_per_step = float(elapsed.item()) / args.steps
        assert bool(torch.isfinite(y).all())
        # end to end: pinned host x in, y back out, every step
        e2e_steps = max(1, min(args.steps, 50))
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            x.copy_(pinned_x, non_blocking=True)
            y = step()
            pinned_y.copy_(y, non_blocking=True)
            stream.synchronize()
        e2e = torch.tensor([time.perf_counter() - t0], device="cuda")
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
        # distinct experts per layer over all ranks (weight bytes actually touched)
        ids = torch.stack([layer.ids for layer in layers]).to(torch.int64)        # [L, per, k]
        gathered = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        distinct = float(sum(len(torch.unique(torch.cat([g[l] for g in gathered]))) for l in range(n_layers)))
    if rank == 0:
        hbm_peak, peak_kind = peaks()
        layouts = specs[0].layouts()
        expert_bytes = layouts[1].expert_bytes + layouts[2].expert_bytes + layouts[3].expert_bytes
        replicated = layouts[0].tensor_bytes + layouts[7].tensor_bytes + sum(layouts[i].tensor_bytes for i in (4, 5, 6))
        touched = distinct * expert_bytes + n_layers * world * replicated
        us = ms_per_step * 1e3 / (tokens * n_layers)
        achieved = touched / (ms_per_step * 1e-3) / 1e9
        print(json.dumps({
            "metric": "moe_layer_us_per_token_decode", "value": us, "unit": "us/token", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"c4: batched decode, 64 sequences x 1 token through {n_layers} Q4_K layers, Zipf(1.1) expert popularity",
                       "tokens_per_step": tokens, "layers": n_layers,
                       "parallelism": f"expert parallel, {epr} experts per GPU, router and shared expert replicated, tokens data-parallel",
                       "exchange": "torch.distributed all_to_all_single over NCCL, two per layer (rows with their expert ids, outputs); the shared expert runs on a second stream under the exchange",
                       "same_workload_on_one_gpu": "python bench.py --workload c4 (no exchange; 174 us per layer measured)",
                       "router": args.router, "l2": f"{n_layers} layers of weights per step ({touched / world / 1e6:.0f} MB per GPU), L2 is 126 MB",
                       "distinct_experts_per_layer": distinct / n_layers},
            "roofline": {"bound": "hbm", "kernel": "whole step, all GPUs", "achieved": achieved, "peak": hbm_peak * world, "unit": "GB/s",
                         "frac": achieved / (hbm_peak * world), "peak_kind": peak_kind, "traffic": None, "algorithmic_bytes": touched,
                         "kernel_us": ms_per_step * 1e3},
            "e2e": {"value": float(e2e.item()) / e2e_steps * 1e6 / (tokens * n_layers), "unit": "us/token",
                    "h2d_bytes_per_step": int(pinned_x.numel() * 4 * world), "d2h_bytes_per_step": int(pinned_y.numel() * 4 * world),
                    "steps": e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks.summary(), "cpu_baseline": None,
        }))
    for layer in layers:
        layer.close()
    lib.qw4cu_set_stream(None)
    dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=400)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c1")
    parser.add_argument("--layers", type=int, default=8, help="rotating weight sets (L2 hygiene)")
    parser.add_argument("--router", default="exact", choices=["exact", "fast"])
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--expert-path", type=int, default=-1, help="-1 auto, 0 CUDA-core kernels, 1 tensor-core grouped kernels")
    parser.add_argument("--tile-path", type=int, default=-1, help="-1 auto, 0 never, 1 tile kernels for every batch of more than four rows")
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--ep-layers", type=int, default=48, help="layers of the expert-parallel workload (N > 1)")
    parser.add_argument("--profile", action="store_true",
                        help="only W + K directly launched steps (the command to run under ncu); prints no bench line")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    hbm_peak, peak_kind = peaks()

    if args.impl == "reference":
        if rank != 0:
            return
        # N > 1 runs the sharded batched-decode workload (c4): the CPU arm times the same 64-token batch through one of
        # its layers on the host cores (a bounded sample: every layer costs the same)
        name = "c4" if world > 1 and args.workload == "c1" else args.workload
        desc, tokens, specs, x = workload(name, 1)
        if name == "c4":
            desc = "c4: batched decode, 64 sequences x 1 token through Q4_K layers, Zipf(1.1) expert popularity (CPU: one layer sampled)"
        per_step = 0.6 * tokens / max(1, min(tokens, len(os.sched_getaffinity(0))))
        steps = max(1, min(args.steps, int(120 / max(per_step, 1e-3))))
        seconds, threads, kind = cpu_reference_step(specs, x, steps, min(args.warmup, 3))
        us_per_token = seconds * 1e6 / tokens
        unit = "us/token"
        print(json.dumps({
            "impl": "reference", "metric": "moe_layer_us_per_token_decode", "value": us_per_token, "unit": unit,
            "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": seconds * 1e3,
            "higher_is_better": False, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc, "tokens_per_step": tokens},
            "cpu_baseline": {"value": us_per_token, "unit": unit, "cores": threads, "kind": kind,
                             "sample": f"{steps} steps of the full {tokens}-token batch through one layer"},
            "e2e": {"value": us_per_token, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    if world > 1:
        return run_expert_parallel(args, rank, local_rank, world)

    api = abi.product()
    lib = api.lib
    if lib.qw4cu_device_count() <= 0:
        raise SystemExit(f"no CUDA device: {lib.qw4cu_last_error().decode()}")
    if lib.qw4cu_set_device(local_rank) != 0:
        raise SystemExit(lib.qw4cu_last_error().decode())
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    lib.qw4cu_set_router_mode(1 if args.router == "fast" else 0)
    lib.qw4cu_set_tile_path(args.tile_path)
    lib.qw4cu_set_expert_path(args.expert_path)
    desc, tokens, specs, x = workload(args.workload, args.layers)
    layers = [MoeLayer(api, spec, tokens) for spec in specs]
    err = abi.Qwen4Error()
    x_dev = lib.qw4cu_malloc(x.nbytes)
    y_dev = [lib.qw4cu_malloc(x.nbytes) for _ in layers]
    assert lib.qw4cu_upload(x_dev, x.ctypes.data, x.nbytes) == 0

    def device_step(i):
        layer = layers[i % len(layers)]
        st = lib.qw4cu_moe_forward_device(layer.moe, x_dev, y_dev[i % len(layers)], tokens, None, None, layer.work, C.byref(err))
        if st:
            raise abi.MoeError(st, err)

    def sync_all():
        for layer in layers:
            st = lib.qw4cu_moe_work_sync(layer.work, C.byref(err))
            if st:
                raise abi.MoeError(st, err)

    def barrier():
        if dist is not None:
            dist.barrier()

    if args.profile:
        lib.qw4cu_set_graph_mode(0)
        for i in range(args.warmup + args.steps):
            device_step(i)
        sync_all()
        print(json.dumps({"profile_steps": args.steps, "warmup": args.warmup,
                          "launches": int(lib.qw4cu_launch_count())}))
        return

    # routes of every layer (for byte counts) and a first correctness-preserving pass
    ids_per_layer = []
    for layer in layers:
        _, ids, _ = layer.forward(x)
        ids_per_layer.append(ids)

    # ---- per-kernel times (events between kernels), untimed for the headline --------------------
    lib.qw4cu_set_graph_mode(0)
    lib.qw4cu_set_stage_timing(1)
    for i in range(3 * len(layers)):
        device_step(i)
    sync_all()
    stage_ms = (C.c_double * len(STAGES))()
    forwards = C.c_uint64()
    lib.qw4cu_stage_times(stage_ms, C.byref(forwards))           # discard the warm-up passes
    profile_steps = max(len(layers) * 4, min(args.steps, 200))
    for i in range(profile_steps):
        device_step(i)
    sync_all()
    lib.qw4cu_stage_times(stage_ms, C.byref(forwards))
    lib.qw4cu_set_stage_timing(0)
    stage_us = {name: stage_ms[j] * 1e3 / max(forwards.value, 1) for j, name in enumerate(STAGES)}
    bytes_by_stage = {name: 0.0 for name in STAGES}
    distinct = 0.0
    for spec, ids in zip(specs, ids_per_layer):
        sb, d = stage_bytes(spec, ids)
        distinct += d / len(specs)
        for name in STAGES:
            bytes_by_stage[name] += sb[name] / len(specs)
    dominant = max(STAGES, key=lambda name: stage_us[name])

    # ---- headline: K steps, device resident, CUDA events on the launching stream -----------------
    lib.qw4cu_set_graph_mode(0 if args.no_graph else 1)
    launches_before_warm = lib.qw4cu_launch_count()
    spin_until = time.perf_counter() + 0.3                       # let clocks settle (untimed)
    i = 0
    while time.perf_counter() < spin_until or i < 3 * len(layers):
        device_step(i)
        i += 1
        if i % 64 == 0:
            sync_all()
    for j in range(args.warmup):
        device_step(i + j)
    sync_all()
    barrier()
    first = layers[0]
    with ClockSampler(local_rank) as clocks:
        launches_before = lib.qw4cu_launch_count()
        lib.qw4cu_moe_work_timer_begin(first.work)
        for j in range(args.steps):
            device_step(j)
        lib.qw4cu_moe_work_timer_end(first.work)
        elapsed_ms = lib.qw4cu_moe_work_timer_elapsed_ms(first.work)
        sync_all()
        launches = lib.qw4cu_launch_count() - launches_before
        # keep the GPU loaded a little longer so that short timed regions still get clock samples
        extra_until = time.perf_counter() + 0.05
        j = 0
        while time.perf_counter() < extra_until:
            device_step(j)
            j += 1
        sync_all()
    barrier()
    if dist is not None:
        import torch
        t = torch.tensor([elapsed_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    us_per_token = ms_per_step * 1e3 / (tokens * world)          # whole job: world replicas of the batch

    # ---- end to end through the reference-facing host API ------------------------------------------
    lib.qw4cu_set_graph_mode(0)
    pinned = lib.qw4cu_host_alloc(2 * x.nbytes)
    x_host = np.ctypeslib.as_array(C.cast(pinned, C.POINTER(C.c_float)), shape=(2 * x.size,))
    x_pin = x_host[:x.size].reshape(x.shape)
    y_pin = x_host[x.size:].reshape(x.shape)
    x_pin[:] = x
    xv, yv = abi.f32_view(x_pin), abi.f32_view(y_pin)

    def host_step(i):
        layer = layers[i % len(layers)]
        st = lib.qwen4_moe_forward(layer.moe, xv, yv, None, layer.work, C.byref(err))
        if st:
            raise abi.MoeError(st, err)

    e2e_steps = min(args.steps, 400)
    for i in range(max(args.warmup, len(layers))):
        host_step(i)
    barrier()
    start = time.perf_counter()
    for i in range(e2e_steps):
        host_step(i)
    e2e_seconds = time.perf_counter() - start
    barrier()
    if dist is not None:
        import torch
        t = torch.tensor([e2e_seconds], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    e2e_us_per_token = e2e_seconds / e2e_steps * 1e6 / (tokens * world)

    if rank != 0:
        return

    # ---- CPU baseline (rank 0, N = 1 only) ----------------------------------------------------------
    cpu = None
    if world == 1:
        guess = 0.6 * tokens / max(1, min(tokens, len(os.sched_getaffinity(0))))
        repeats = max(1, int(args.cpu_seconds / max(guess, 1e-3)))
        seconds, threads, kind = cpu_reference_step(specs, x, repeats, 1)
        cpu = {"value": seconds * 1e6 / tokens, "unit": "us/token", "cores": threads, "kind": kind,
               "sample": f"{repeats} passes of the full {tokens}-token batch through layer 0, "
                         f"tokens sharded over {threads} threads"}

    layer_bytes = sum(bytes_by_stage.values())
    layer_gbs = layer_bytes / (ms_per_step * 1e-3) / 1e9
    phases = None
    if launches == args.steps:
        # one launch per step: the whole layer ran as the one-kernel decode path.  Its duration is the
        # event-timed step (launch gaps included, so the fraction is a lower bound) and its algorithmic
        # bytes are every weight byte the step must read once.
        dominant = "fused_decode_kernel"
        kernel_us, kernel_bytes = ms_per_step * 1e3, layer_bytes
        clocks16 = (C.c_uint64 * 16)()
        lib.qw4cu_decode_phase_clocks(layers[(args.steps - 1) % len(layers)].work, clocks16)
        ticks = [int(v) for v in clocks16[:13]]
        names = ["stage_x", "fast_logits", "digitise_x", "barrier_1", "speculate_sets", "list_experts", "gate_up_slices",
                 "store_digits", "barrier_2_and_routes", "verify_routes", "load_act_digits", "down_combine"]
        phases = {name: ticks[j + 1] - ticks[j] for j, name in enumerate(names)}
        phases["unit"] = "SM cycles of the first streaming CTA, last timed launch"
    else:
        kernel_us, kernel_bytes = stage_us[dominant], bytes_by_stage[dominant]
    achieved = kernel_bytes / (kernel_us * 1e-6) / 1e9 if kernel_us > 0 else 0.0
    tensor = None
    if args.workload in ("c2", "c3"):
        # FLOPs of the chunk (routed 2 * pairs * 3 * H * I, shared, router) against the measured dense bf16 rate
        spec0 = specs[0]
        pairs = tokens * spec0.top_k
        flops = 2.0 * pairs * 3 * spec0.hidden * spec0.inter + 2.0 * tokens * 3 * spec0.hidden * spec0.shared_inter \
            + 2.0 * tokens * spec0.hidden * (spec0.experts + 1)
        peak_tf = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()).get("bf16_tflops_sustained", 1422.1) \
            if (ROOT / "MEASURED_PEAKS.json").exists() else 1400.0
        tensor = {"bound": "tensor", "flop_per_step": flops, "achieved": flops / (ms_per_step * 1e-3) / 1e12, "peak": peak_tf,
                  "unit": "TFLOP/s", "frac": flops / (ms_per_step * 1e-3) / 1e12 / peak_tf,
                  "note": "whole step against the sustained dense bf16 rate; at about 20 rows per expert the binding roof is HBM"}
    traffic = TRAFFIC.get(f"{args.workload}:{dominant}")
    line = {
        "metric": "moe_layer_us_per_token_decode" if args.workload not in ("c2", "c3") else "moe_layer_us_per_token_prefill",
        "value": us_per_token, "unit": "us/token", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "tokens_per_step": tokens, "parallelism": "single GPU" if world == 1 else f"{world} replicas",
                   "router": args.router, "launch": "one persistent kernel per layer" if phases else ("direct" if args.no_graph else "cuda-graph replay per layer"),
                   "l2": f"rotating {len(layers)} weight sets ({layer_bytes * len(layers) / 1e6:.0f} MB touched between reuse of a set; L2 is 126 MB)",
                   "distinct_experts_per_step": distinct, "spinup_ms": 300},
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": traffic,
                     "algorithmic_bytes": kernel_bytes, "kernel_us": kernel_us},
        "roofline_tensor": tensor,
        "phases": phases,
        "tokens_per_s": tokens * world / (ms_per_step * 1e-3),
        "layer": {"weight_bytes": layer_bytes, "achieved_gbs": layer_gbs, "frac_of_measured_peak": layer_gbs / hbm_peak,
                  "frac_of_nominal_8tbs": layer_gbs / NOMINAL_HBM_GBS,
                  "stage_us_multi_kernel_path": stage_us, "stage_bytes": bytes_by_stage},
        "e2e": {"value": e2e_us_per_token, "unit": "us/token", "h2d_bytes_per_step": int(x.nbytes),   # status words: cleared only after an error
                "d2h_bytes_per_step": int(x.nbytes) + 16, "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
