#!/usr/bin/env python
"""Benchmark of the B200 Qwen4 MoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c0|c1|c2|c3|c4] [--sharded c4,c3] [--impl reference]

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

With N > 1 (torchrun, one rank per GPU) every rank runs its own replica of that batch (single-token
decode stays on one GPU: independent replicas, no collective on the data path, weak scaling).

The two sharded configurations are measured beside it at every N, N = 1 included, through the
library's expert-parallel step (`qw4cu_moe_ep_forward_device`: experts in N contiguous blocks, one
all-gather and one reduce-scatter per layer, by the library's push / pull kernels over NVLink peer memory
or through NCCL), and reported under "sharded": c4 (64
streams x 1 token through 48 Q4_K layers, Zipf expert popularity) and c3 (8 chunks of 1024 tokens
through 48 layers, Q2_K routed + Q4_K shared), each with the parity of its first layer against the
CPU oracle.  `--workload c3|c4` runs one of them alone; `--sharded ""` leaves them out.  At N = 1 the
line also carries the single-token step ("c0"), the 1024-token prefill chunk ("c2") and the 1 + 3-row
verify append through a 48-layer stack ("verify_stack").
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel.  ncu cannot run inside a timed
# benchmark, so the figure comes from the capture summarised in the named file (same command, same workload) and
# is reported with that source; a workload without a capture of its current kernel reports null.
TRAFFIC = {
    "c1:fused_decode_kernel": {"bytes": 64.77e6 + 1.68e6, "source": "profiles/decode_c1_fused_decode_kernel.md"},
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
    elif name == "c3-layer":
        specs = [synth.make_layer(3, layer=l, routed_type=abi.Q2_K, shared_type=abi.Q4_K) for l in range(layers)]
        x = synth.activations(3, 1024)
        desc = "c3 (one GPU): 1024-token prefill chunk, Q2_K routed + Q4_K shared, uniform routing"
    elif name == "c4-layer":
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


# ---- sharded workloads (expert parallel over the ranks of this job, world 1 included) -----------------
SHARDED = {
    # name: (routed type, shared type, tokens per chunk, chunks, Zipf-skewed router, seed, description)
    "c4": (abi.Q4_K, abi.Q4_K, 64, 1, True, 4, "c4: batched decode, 64 sequences x 1 token through {layers} Q4_K layers, Zipf(1.1) expert popularity"),
    "c3": (abi.Q2_K, abi.Q4_K, 1024, 8, False, 3, "c3: 8192-token prefill (8 chunks of 1024) through {layers} layers, Q2_K routed + Q4_K shared, uniform routing"),
}


def run_sharded(name, args, api, rank, world, control, hbm_peak, peak_kind):
    """One sharded workload through qw4cu_moe_ep_forward_device: experts in `world` contiguous blocks, tokens
    data-parallel, one all-gather and one reduce-scatter per layer issued by the library over NCCL.  The same
    code path runs at world 1 (the collectives become copies), so the numbers of all N are one curve.  Layer 0
    holds quantised Gaussian weights and is checked against the CPU oracle on a token sample; the other layers
    hold fabricated blocks (same shapes and byte counts).  Every layer reads the same resident chunk of
    activations (in the engine the MoE input comes from the layer's own mixer, not from the previous MoE)."""
    from picoforge_b200.expert_parallel import Communicator, EpLayer
    lib = api.lib
    routed, shared, chunk_tokens, chunks, skewed, seed, text = SHARDED[name]
    n_layers = args.ep_layers
    per, epr = chunk_tokens // world, 512 // world
    broadcast = None
    if world > 1:
        def broadcast(payload):
            box = [payload]
            control.broadcast_object_list(box, src=0)
            return box[0]
    comm = Communicator(api, rank, world, broadcast)
    x_all = synth.activations(seed, chunk_tokens * chunks)
    if skewed:
        x_all[:, 0] = 1.0
    layers, spec = [], None
    for l in range(n_layers):
        spec = synth.make_layer(seed, layer=l, routed_type=routed, shared_type=shared, shard=(rank * epr, epr) if world > 1 else None,
                                fabricated=l > 0, reuse=spec if l > 1 else None)
        if skewed:
            synth.zipf_router_bias(spec, seed + l)
        layers.append(EpLayer(api, spec, per, world, rank))
    layouts = spec.layouts()
    expert_bytes = layouts[1].expert_bytes + layouts[2].expert_bytes + layouts[3].expert_bytes
    replicated = layouts[0].tensor_bytes + layouts[7].tensor_bytes + sum(layouts[i].tensor_bytes for i in (4, 5, 6))
    spec.tensors = []
    hidden = 2048
    x_dev = []
    for c in range(chunks):
        rows = np.ascontiguousarray(x_all[c * chunk_tokens + rank * per:c * chunk_tokens + (rank + 1) * per])
        pointer = lib.qw4cu_malloc(rows.nbytes)
        assert lib.qw4cu_upload(pointer, rows.ctypes.data, rows.nbytes) == 0
        x_dev.append(pointer)
    y_dev = lib.qw4cu_malloc(per * hidden * 4)

    def barrier():
        if world > 1:
            control.barrier()

    # ---- parity of layer 0 on this rank's first tokens of chunk 0 (rank 0 reports) ----
    layers[0].forward(comm, x_dev[0], y_dev)
    layers[0].sync()
    parity = None
    if rank == 0:
        import oracle
        sample = min(8, per)
        y0 = np.empty((per, hidden), np.float32)
        assert lib.qw4cu_download(y0.ctypes.data, y_dev, y0.nbytes) == 0
        ids0, _ = layers[0].routes()
        full = synth.make_layer(seed, layer=0, routed_type=routed, shared_type=shared)
        if skewed:
            synth.zipf_router_bias(full, seed)
        want = oracle.forward(full, x_all[:sample], threads=synth.threads())
        parity = {"tokens": sample, "max_abs": float(np.abs(y0[:sample] - want["y"]).max()),
                  "ids_equal": bool(np.array_equal(ids0[:sample], want["ids"]))}
        del full
    barrier()                                                                        # the other ranks wait here while rank 0 runs the oracle

    def step():
        for c in range(chunks):
            for layer in layers:
                layer.forward(comm, x_dev[c], y_dev)

    def sync_all():
        for layer in layers:
            layer.sync()

    lib.qw4cu_set_graph_mode(0 if args.no_graph else 1)                              # per layer and chunk: captured at its second step, replayed after
    for _ in range(max(2, args.ep_warmup)):
        step()
    sync_all()
    barrier()
    work0 = layers[0].layer.work
    before = lib.qw4cu_launch_count()
    lib.qw4cu_moe_work_timer_begin(work0)
    for _ in range(args.ep_steps):
        step()
    lib.qw4cu_moe_work_timer_end(work0)
    elapsed_ms = lib.qw4cu_moe_work_timer_elapsed_ms(work0)
    sync_all()
    launches = lib.qw4cu_launch_count() - before
    barrier()
    # one more, untimed, step with an event at every stage boundary (it synchronises per layer: a profile, not a timing)
    lib.qw4cu_set_graph_mode(0)
    lib.qw4cu_ep_trace(1)
    step()
    stage_ms = (C.c_double * 10)()
    traced = lib.qw4cu_ep_trace_read(stage_ms, 10)
    lib.qw4cu_ep_trace(0)
    stage_names = ["router_logits", "route_pack", "all_gather", "local_ids_lists", "digits_x", "gate_up", "digits_act", "down",
                   "shared_join_partial_sums", "reduce_scatter"]
    stages_us = {n: stage_ms[i] * 1e3 / max(traced, 1) for i, n in enumerate(stage_names)}
    barrier()
    distinct = None
    if chunks == 1:                                                                   # decode: the experts actually touched, over all ranks
        ids_local = np.stack([layer.routes()[0] for layer in layers])                 # [L, per, k]
        gathered = [ids_local]
        if world > 1:
            gathered = [None] * world
            control.all_gather_object(gathered, ids_local)
        distinct = float(sum(len(np.unique(np.concatenate([g[l] for g in gathered]))) for l in range(n_layers)))
    if world > 1:
        import torch
        t = torch.tensor([elapsed_ms], dtype=torch.float64)
        control.all_reduce(t, op=control.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    transport = "this library's kernels over NVLink peer memory (push all-gather, pull reduce-scatter)" if lib.qw4cu_ep_transport(comm.handle) \
        else ("none (one rank)" if world == 1 else "NCCL (ncclAllGather, ncclReduceScatter)")
    for layer in layers:
        layer.close()
    barrier()
    comm.close()
    for pointer in x_dev + [y_dev]:
        lib.qw4cu_free(pointer)
    if rank != 0:
        return None
    ms_per_step = elapsed_ms / args.ep_steps
    tokens = chunk_tokens * chunks
    passes = chunks * n_layers                                                        # chunk-layers per step
    if distinct is None:
        touched = passes * (512 * expert_bytes + world * replicated)                  # prefill: every expert of every layer, per chunk
    else:
        touched = distinct * expert_bytes + n_layers * world * replicated
    achieved = touched / (ms_per_step * 1e-3) / 1e9
    out = {
        "workload": text.format(layers=n_layers), "n_gpus": world, "steps": args.ep_steps, "warmup": max(2, args.ep_warmup), "launch": "direct" if args.no_graph else "cuda-graph replay per layer and chunk (collectives captured)",
        "ms_per_step": ms_per_step, "us_per_token_layer": ms_per_step * 1e3 / (tokens * n_layers),
        "us_per_chunk_layer": ms_per_step * 1e3 / passes, "tokens_per_s": tokens / (ms_per_step * 1e-3), "scaling": "strong",
        "parallelism": f"expert parallel over {world} GPU(s): {epr} experts each, router and shared expert replicated, tokens data-parallel; "
                       "per layer one all-gather of token rows and one reduce-scatter of partial sums, issued by the library",
        "transport": transport,
        "weights": "layer 0: quantised Gaussian masters (checked against the CPU oracle); other layers: fabricated blocks of the same formats",
        "roofline": {"bound": "hbm", "kernel": "whole step, all GPUs", "achieved": achieved, "peak": hbm_peak * world, "unit": "GB/s",
                     "frac": achieved / (hbm_peak * world), "peak_kind": peak_kind, "algorithmic_bytes": touched, "traffic": None},
        "parity": parity, "gpu_launches": int(launches),
        "stages_us_per_chunk_layer_rank0": stages_us,
    }
    if distinct is not None:
        out["distinct_experts_per_layer"] = distinct / n_layers
    else:
        flops = passes * (2.0 * chunk_tokens * 10 * 3 * 2048 * 512 + 2.0 * chunk_tokens * 3 * 2048 * 512 + 2.0 * chunk_tokens * 2048 * 513)
        peak_tf = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()).get("bf16_tflops_sustained", 1422.1) \
            if (ROOT / "MEASURED_PEAKS.json").exists() else 1400.0
        out["roofline_tensor"] = {"bound": "tensor", "achieved": flops / (ms_per_step * 1e-3) / 1e12, "peak": peak_tf * world, "unit": "TFLOP/s",
                                  "frac": flops / (ms_per_step * 1e-3) / 1e12 / (peak_tf * world),
                                  "note": "against the sustained dense bf16 rate; at about 20 rows per expert the binding roof is HBM"}
    return out


# ---- main --------------------------------------------------------------------------------------
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c1", help="c0 | c1 | c2 | c3-layer | c4-layer (one layer, every rank runs its own replica); c3 | c4: only that sharded workload")
    parser.add_argument("--layers", type=int, default=8, help="rotating weight sets (L2 hygiene)")
    parser.add_argument("--router", default="exact", choices=["exact", "fast"])
    parser.add_argument("--repeats", type=int, default=25, help="timed regions of --steps steps each; the value is their median")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--expert-path", type=int, default=-1, help="-1 auto, 0 CUDA-core kernels, 1 tensor-core grouped kernels")
    parser.add_argument("--tile-path", type=int, default=-1, help="-1 auto, 0 never, 1 tile kernels for every batch of more than four rows")
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--sharded", default="c4,c3", help="sharded workloads measured beside the headline (comma list, '' for none)")
    parser.add_argument("--ep-layers", type=int, default=48, help="layers of the sharded workloads")
    parser.add_argument("--ep-steps", type=int, default=3)
    parser.add_argument("--ep-warmup", type=int, default=1)
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
        name = args.workload if args.workload in ("c0", "c1", "c2") else "c1"
        desc, tokens, specs, x = workload(name, 1)
        per_step = 0.6 * tokens / max(1, min(tokens, len(os.sched_getaffinity(0))))
        steps = max(1, min(args.steps, int(120 / max(per_step, 1e-3))))
        seconds, threads, kind = cpu_reference_step(specs, x, steps, min(args.warmup, 3))
        us_per_token = seconds * 1e6 / tokens
        unit = "us/token"
        print(json.dumps({
            "impl": "reference", "metric": "moe_layer_us_per_token_decode" if name != "c2" else "moe_layer_us_per_token_prefill",
            "value": us_per_token, "unit": unit,
            "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": seconds * 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc, "tokens_per_step": tokens},
            "cpu_baseline": {"value": us_per_token, "unit": unit, "cores": threads, "kind": kind,
                             "sample": f"{steps} steps of the full {tokens}-token batch through one layer"},
            "e2e": {"value": us_per_token, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    api = abi.product()
    lib = api.lib
    if lib.qw4cu_device_count() <= 0:
        raise SystemExit(f"no CUDA device: {lib.qw4cu_last_error().decode()}")
    if lib.qw4cu_set_device(local_rank) != 0:
        raise SystemExit(lib.qw4cu_last_error().decode())
    control = None
    if world > 1:
        import torch.distributed as control                                         # gloo: the control plane only (ids, barriers, maxima)
        control.init_process_group("gloo")

    lib.qw4cu_set_router_mode(1 if args.router == "fast" else 0)
    lib.qw4cu_set_tile_path(args.tile_path)
    lib.qw4cu_set_expert_path(args.expert_path)
    sharded_names = [n for n in args.sharded.split(",") if n]
    if args.workload in SHARDED:
        sharded_names, headline = [args.workload], None
    else:
        headline = decode_line(args, api, rank, local_rank, world, control, hbm_peak, peak_kind)
        if not args.profile and args.workload == "c1" and world == 1:
            # the single-token figure rides on the same line (five regions are enough for a side figure; no CPU pass)
            import copy
            side = copy.copy(args)
            side.workload, side.repeats, side.cpu_seconds = "c0", 5, 0.0
            c0 = decode_line(side, api, rank, local_rank, world, control, hbm_peak, peak_kind)
            headline["c0"] = {"workload": c0["config"]["workload"], "us_per_layer": c0["ms_per_step"] * 1e3, "roofline": c0["roofline"],
                              "e2e": c0["e2e"], "timing": c0["timing"], "gpu_launches": c0["gpu_launches"]}
            # ... and so does the 1024-token prefill chunk (two weight sets, three regions of at most five steps)
            side = copy.copy(args)
            side.workload, side.repeats, side.cpu_seconds, side.layers, side.steps = "c2", 3, 0.0, 2, min(args.steps, 5)
            c2 = decode_line(side, api, rank, local_rank, world, control, hbm_peak, peak_kind)
            headline["c2"] = {"workload": c2["config"]["workload"], "us_per_chunk": c2["ms_per_step"] * 1e3, "us_per_token": c2["value"],
                              "roofline": c2["roofline"], "roofline_tensor": c2["roofline_tensor"], "timing": c2["timing"],
                              "stage_us": c2["layer"]["stage_us_multi_kernel_path"], "gpu_launches": c2["gpu_launches"]}
    if args.profile:
        return
    sharded = {}
    for name in sharded_names:
        result = run_sharded(name, args, api, rank, world, control, hbm_peak, peak_kind)
        if rank == 0:
            sharded[name] = result
    if control is not None:
        control.barrier()
        control.destroy_process_group()
    if rank != 0:
        return
    if headline is None:                                                             # a sharded workload on its own
        only = sharded[sharded_names[0]]
        headline = {"metric": "moe_layer_us_per_token_" + ("decode" if sharded_names[0] == "c4" else "prefill"),
                    "value": only["us_per_token_layer"], "unit": "us/token", "n_gpus": world, "steps": only["steps"], "warmup": only["warmup"],
                    "ms_per_step": only["ms_per_step"], "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                    "data": "synthetic", "config": {"workload": only["workload"], "parallelism": only["parallelism"]},
                    "roofline": only["roofline"], "e2e": None, "gpu_launches": only["gpu_launches"], "cpu_baseline": None}
    headline["sharded"] = sharded
    print(json.dumps(headline))


def decode_line(args, api, rank, local_rank, world, control, hbm_peak, peak_kind):
    """The single-layer workloads (c0, c1, c2): every rank runs its own replica of the batch on its GPU (independent
    layers, no collective on the data path: weak scaling); rank 0 returns the JSON line, the others None."""
    lib = api.lib
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
        if control is not None:
            control.barrier()

    def max_over_ranks(value):
        if control is None:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64)
        control.all_reduce(t, op=control.ReduceOp.MAX)
        return float(t.item())

    if args.profile:
        lib.qw4cu_set_graph_mode(0)
        for i in range(args.warmup + args.steps):
            device_step(i)
        sync_all()
        print(json.dumps({"profile_steps": args.steps, "warmup": args.warmup,
                          "launches": int(lib.qw4cu_launch_count())}))
        return None

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
    region_ms = []
    with ClockSampler(local_rank) as clocks:
        launches_before = lib.qw4cu_launch_count()
        for _ in range(max(1, args.repeats)):                     # the reference's protocol: repeated regions, median and spread
            lib.qw4cu_moe_work_timer_begin(first.work)
            for j in range(args.steps):
                device_step(j)
            lib.qw4cu_moe_work_timer_end(first.work)
            region_ms.append(lib.qw4cu_moe_work_timer_elapsed_ms(first.work))
        sync_all()
        launches = (lib.qw4cu_launch_count() - launches_before) // max(1, args.repeats)
    barrier()
    region_ms = sorted(region_ms)
    elapsed_ms = max_over_ranks(float(np.median(region_ms)))
    ms_per_step = elapsed_ms / args.steps
    us_per_token = ms_per_step * 1e3 / (tokens * world)          # whole job: world replicas of the batch
    spread = {"regions": len(region_ms), "steps_per_region": args.steps,
              "p10_ms_per_step": region_ms[len(region_ms) // 10] / args.steps, "p90_ms_per_step": region_ms[(len(region_ms) * 9) // 10] / args.steps}

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
    e2e_seconds = max_over_ranks(time.perf_counter() - start)
    barrier()
    e2e_us_per_token = e2e_seconds / e2e_steps * 1e6 / (tokens * world)

    clocks16 = (C.c_uint64 * 16)()
    lib.qw4cu_decode_phase_clocks(layers[(args.steps - 1) % len(layers)].work, clocks16)

    # ---- the batch's real caller: speculative verify of 1 + 3 rows through a 48-layer stack (host buffers, one wait) ----
    stack = None
    if tokens <= 4 and world == 1 and not args.profile:
        depth = 48
        handles = (C.c_void_p * depth)(*[layers[i % len(layers)].moe for i in range(depth)])
        cfg = specs[0].config()
        verify = C.c_void_p()
        if lib.qw4cu_verify_create(handles, depth, C.byref(cfg), C.byref(verify), C.byref(err)) == 0:
            xs, ys = np.ascontiguousarray(x[:tokens]), np.empty_like(x[:tokens])
            appends = 12
            for i in range(3 + appends):
                if i == 3:
                    start = time.perf_counter()
                # every layer's output feeds the next: keep the chain finite by restarting from x each append
                if lib.qw4cu_verify_append(verify, xs.ctypes.data, tokens, ys.ctypes.data, None, C.byref(err)) != 0:
                    raise abi.MoeError(err.code, err)
                lib.qw4cu_verify_keep(verify, 1, C.byref(err))
            seconds = (time.perf_counter() - start) / appends
            lib.qw4cu_verify_destroy(verify)
            stack = {"layers": depth, "rows": tokens, "ms_per_append": seconds * 1e3, "us_per_layer": seconds * 1e6 / depth,
                     "us_per_token_layer": seconds * 1e6 / depth / tokens,
                     "note": "qw4cu_verify_append: host x in, host y out, 48 layers enqueued back to back, one host wait; "
                             "the 8 weight sets repeat down the stack"}
    for layer in layers:
        layer.close()
    for pointer in [x_dev] + y_dev:
        lib.qw4cu_free(pointer)
    if rank != 0:
        return None

    # ---- CPU baseline (rank 0, N = 1 only) ----------------------------------------------------------
    cpu = None
    if world == 1 and args.cpu_seconds > 0:
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
        ticks = [int(v) for v in clocks16[:13]]
        names = ["stage_x", "fast_logits", "digitise_x", "barrier_1", "speculate_sets", "list_experts", "gate_up_slices",
                 "store_digits", "barrier_2_and_routes", "verify_routes", "load_act_digits", "down_combine"]
        phases = {name: ticks[j + 1] - ticks[j] for j, name in enumerate(names)}
        phases["unit"] = "SM cycles of the first streaming CTA, last timed launch"
    else:
        kernel_us, kernel_bytes = stage_us[dominant], bytes_by_stage[dominant]
    achieved = kernel_bytes / (kernel_us * 1e-6) / 1e9 if kernel_us > 0 else 0.0
    tensor = None
    if args.workload in ("c2", "c3-layer"):
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
    clock_summary = clocks.summary()
    line = {
        "metric": "moe_layer_us_per_token_decode" if args.workload not in ("c2", "c3-layer") else "moe_layer_us_per_token_prefill",
        "value": us_per_token, "unit": "us/token", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "tokens_per_step": tokens, "parallelism": "single GPU" if world == 1 else f"{world} GPUs, one independent replica of the batch each (no collective on the data path)",
                   "router": args.router, "launch": "one persistent kernel per layer" if phases else ("direct" if args.no_graph else "cuda-graph replay per layer"),
                   "l2": f"rotating {len(layers)} weight sets ({layer_bytes * len(layers) / 1e6:.0f} MB touched between reuse of a set; L2 is 126 MB)",
                   "distinct_experts_per_step": distinct, "spinup_ms": 300},
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "peak_kind": peak_kind, "traffic": traffic["bytes"] if traffic else None,
                     "traffic_source": traffic["source"] if traffic else None,
                     "algorithmic_bytes": kernel_bytes, "kernel_us": kernel_us},
        "timing": dict(spread, median_ms_per_step=ms_per_step,
                       ms_per_step_x_sm_mhz=ms_per_step * clock_summary["sm_mhz"] if clock_summary["sm_mhz"] else None),
        "roofline_tensor": tensor,
        "phases": phases,
        "tokens_per_s": tokens * world / (ms_per_step * 1e-3),
        "layer": {"weight_bytes": layer_bytes, "achieved_gbs": layer_gbs, "frac_of_measured_peak": layer_gbs / hbm_peak,
                  "frac_of_nominal_8tbs": layer_gbs / NOMINAL_HBM_GBS,
                  "stage_us_multi_kernel_path": stage_us, "stage_bytes": bytes_by_stage},
        "e2e": {"value": e2e_us_per_token, "unit": "us/token", "h2d_bytes_per_step": int(x.nbytes),   # status words: cleared only after an error
                "d2h_bytes_per_step": int(x.nbytes) + 16, "steps": e2e_steps},
        "verify_stack": stack,
        "gpu_launches": int(launches),
        "clocks": clock_summary,
        "cpu_baseline": cpu,
    }
    return line


if __name__ == "__main__":
    main()
