#!/usr/bin/env python3
"""Benchmark of the W4A16 decode GEMV on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1, and each rank's replica for N > 1): the Llama-3-8B decode layer set at M = 1 --
bf16 activations, uint4 weights in ARC packets, group 128, bf16 scale/offset -- i.e. the four
GEMVs qkv (6144x4096), o_proj (4096x4096), gate_up (28672x4096), down_proj (4096x14336) of one
decoder layer, for 32 layers with distinct weights (3.7 GB, far larger than L2, so every call
streams its weights from HBM). One *step* is one pass over all 128 GEMVs. Data is synthetic:
seeded shapes and value distributions, no checkpoint.

The step is captured once as a CUDA graph of 128 launches of the library's C-ABI entry point
(`fk_w4a16_gemv`) and replayed; timing is by CUDA events on the launching stream between a barrier
and a device synchronisation, maximum over ranks. One JSON line is printed by rank 0.

`e2e` measures the same work through the C-ABI entry point that takes HOST buffers
(`fk_w4a16_gemv_host`), one call per GEMV: every call copies its activations from pinned host
memory to the device and its result back inside the timed region.

`--impl reference` times the reference's CPU-runnable arithmetic for this path -- its torch
expression `_explicit_reference_output`, restated in C in oracle/ -- on the host cores, on the same
layer set. (The reference's FK_ENABLE_CUDA=OFF build contains no W4A16 arithmetic at all.)
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "fast-kernels_b200" / "src"))
sys.path.insert(0, str(REPO))

METRIC = "W4A16 GEMV achieved HBM TB/s at M=1 (us/call alongside)"
UNIT = "TB/s"
NUM_LAYERS = 32
FALLBACK_HBM_GBS = 6650.0


def _measured_peak() -> tuple[float, str]:
    path = REPO / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[device_index]) if visible else device_index
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._handle = None

    def _run(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self) -> "ClockSampler":
        if self._handle is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc: object) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz or None,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def _layer_shapes():
    from fast_kernels.workloads import LLAMA3_8B_LAYERS

    return list(LLAMA3_8B_LAYERS)


def _bytes_per_step(shapes) -> int:
    return NUM_LAYERS * sum(s.algorithmic_bytes() for s in shapes)


# ------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's own expression
# ------------------------------------------------------------------------------------------
def _cpu_layer_set(oracle, problems, scratch) -> None:
    for shape, prob in problems:
        oracle.gemv_explicit(prob["activations"], prob["q_u8"], prob["alpha"], prob["beta"],
                             shape.group_size, oracle.BF16, scratch)


def _cpu_problems(oracle):
    import numpy as np
    from fast_kernels.workloads import make_problem

    problems = []
    largest = 0
    for shape in _layer_shapes():
        prob = make_problem(shape)
        problems.append((shape, {
            "activations": oracle.bits_of(prob["activations"]),
            "q_u8": prob["q_u8"].numpy(),
            "alpha": oracle.bits_of(prob["alpha"]),
            "beta": oracle.bits_of(prob["beta"]),
        }))
        largest = max(largest, (shape.n + 1) * shape.k)
    return problems, np.empty(largest, dtype=np.float32)


def run_reference_arm(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import w4a16_oracle as oracle

    shapes = _layer_shapes()
    problems, scratch = _cpu_problems(oracle)
    cores = oracle.num_threads()
    sample_bytes = sum(s.algorithmic_bytes() for s in shapes)  # one decoder layer's four GEMVs
    for _ in range(args.warmup):
        _cpu_layer_set(oracle, problems, scratch)
    start = time.perf_counter()
    for _ in range(args.steps):
        _cpu_layer_set(oracle, problems, scratch)
    elapsed = time.perf_counter() - start
    ms_per_step = elapsed * 1e3 / args.steps
    value = sample_bytes * args.steps / elapsed / 1e12
    sample = ("one decoder layer's 4 GEMVs (qkv, o_proj, gate_up, down_proj) per step: 1/32 of the "
              "GPU arm's step, same shapes and distributions")
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "us_per_call": ms_per_step * 1e3 / len(shapes),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": _config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference's CPU-runnable expression (_explicit_reference_output) restated in C "
                "(oracle/w4a16_oracle.c: oracle_gemv_explicit), all host threads",
    }
    print(json.dumps(line), flush=True)
    return 0


def _config(n_gpus: int) -> dict:
    return {
        "workload": "llama3_8b_decode_layer_set_m1_bf16_g128 x 32 layers (128 GEMV calls per step)",
        "shapes_n_k": [[s.n, s.k] for s in _layer_shapes()],
        "group_size": 128,
        "batch": 1,
        "weights_resident_bytes_per_gpu": _bytes_per_step(_layer_shapes()),
        "l2_policy": "inputs larger than L2: 3.7 GB of distinct weights per step",
        "parallelism": "single GPU" if n_gpus == 1 else f"{n_gpus} independent replicas (no data-path collective)",
        "launch": "one CUDA graph of 128 fk_w4a16_gemv launches per step",
    }


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class LayerSet:
    """Weights (as ARC packets), activations, outputs and scratch for NUM_LAYERS decoder layers."""

    def __init__(self, torch, capi, device) -> None:
        from fast_kernels.workloads import make_problem

        self.torch = torch
        self.capi = capi
        self.lib = capi.load_library()
        self.device = device
        self.calls = []  # (shape, activations, packets, output)
        shapes = _layer_shapes()
        stride = capi.packet_stride_bytes(128)
        base = {}
        for shape in shapes:
            prob = make_problem(shape)
            q, alpha, beta = (prob[key].to(device) for key in ("q_u8", "alpha", "beta"))
            packets = torch.empty(((shape.n // 128) * (shape.k // 128), stride), dtype=torch.uint8,
                                  device=device)
            capi.check(self.lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(),
                                                      packets.data_ptr(), shape.n, shape.k, 128, stride,
                                                      self.stream_ptr()))
            base[shape.name] = (prob["activations"].to(device), packets)
        torch.cuda.synchronize(device)
        gen = torch.Generator(device="cpu").manual_seed(1234)
        for layer in range(NUM_LAYERS):
            for shape in shapes:
                act, packets = base[shape.name]
                if layer > 0:
                    # distinct weights per layer without more host-side generation: a seeded
                    # permutation of whole packets (each keeps its nibbles, scales and offsets)
                    perm = torch.randperm(packets.shape[0], generator=gen).to(device)
                    packets = packets[perm].contiguous()
                out = torch.empty((1, shape.n), dtype=act.dtype, device=device)
                self.calls.append((shape, act, packets, out))
        need = max(int(self.lib.fk_w4a16_workspace_bytes(1, s.n, s.k, 128)) for s in shapes)
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=device)
        self.stride = stride

    def stream_ptr(self) -> int:
        return int(self.torch.cuda.current_stream(self.device).cuda_stream)

    def launch_all(self) -> None:
        """One step: 128 launches on the current stream through the C ABI."""
        stream = self.stream_ptr()
        for shape, act, packets, out in self.calls:
            self.capi.check(self.lib.fk_w4a16_gemv(
                act.data_ptr(), packets.data_ptr(), out.data_ptr(), self.workspace.data_ptr(),
                self.workspace.numel(), 1, shape.n, shape.k, 128, self.stride, self.capi.DTYPE_BF16, stream))

    def capture(self, calls=None):
        torch = self.torch
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        saved = self.calls
        if calls is not None:
            self.calls = calls
        try:
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    self.launch_all()
        finally:
            self.calls = saved
        torch.cuda.current_stream(self.device).wait_stream(side)
        return graph


def _time_graph(torch, graph, reps: int, device) -> float:
    """Seconds for `reps` replays, CUDA events on the current stream."""
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    start.record()
    for _ in range(reps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize(device)
    return start.elapsed_time(stop) / 1e3


NCU_TRAFFIC_RATIO = 1.003


def _e2e(torch, layers: LayerSet, steps: int, device) -> dict:
    """The same step through the C-ABI call that takes HOST buffers (`fk_w4a16_gemv_host`): every
    call copies its activations from pinned host memory to the device, runs the GEMV and copies
    the result back to pinned host memory, all inside the timed region."""
    capi = layers.capi
    lib = layers.lib
    host_in, host_out, dev_in = {}, {}, {}
    for shape, act, _, _ in layers.calls[:4]:
        host_in[shape.name] = act.cpu().pin_memory()
        host_out[shape.name] = torch.empty((1, shape.n), dtype=act.dtype).pin_memory()
        dev_in[shape.name] = torch.empty_like(act)
    h2d = sum(t.numel() * 2 for t in host_in.values()) * NUM_LAYERS
    d2h = sum(t.numel() * 2 for t in host_out.values()) * NUM_LAYERS
    stream = layers.stream_ptr()
    plan = [(host_in[s.name].data_ptr(), packets.data_ptr(), host_out[s.name].data_ptr(),
             dev_in[s.name].data_ptr(), out.data_ptr(), s.n, s.k) for s, _, packets, out in layers.calls]
    ws, ws_bytes = layers.workspace.data_ptr(), layers.workspace.numel()

    def step() -> None:
        for h_in, packets, h_out, d_in, d_out, n, k in plan:
            rc = lib.fk_w4a16_gemv_host(h_in, packets, h_out, d_in, d_out, ws, ws_bytes, 1, n, k, 128,
                                        layers.stride, capi.DTYPE_BF16, stream)
            if rc != 0:
                capi.check(rc)

    step()
    torch.cuda.synchronize(device)
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    host_begin = time.perf_counter()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    host_seconds = time.perf_counter() - host_begin  # time the host spent enqueueing
    torch.cuda.synchronize(device)
    seconds = start.elapsed_time(stop) / 1e3
    # the results are real: the last call's output on the host equals the device tensor
    last_shape, _, _, last_out = layers.calls[-1]
    if not torch.equal(host_out[last_shape.name], last_out.cpu()):
        raise SystemExit("e2e: host result differs from the device result")
    return {"seconds": seconds, "host_seconds": host_seconds, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h}


def _cpu_baseline_leg() -> dict:
    from oracle import w4a16_oracle as oracle

    problems, scratch = _cpu_problems(oracle)
    shapes = _layer_shapes()
    _cpu_layer_set(oracle, problems, scratch)
    reps = 0
    start = time.perf_counter()
    while True:
        _cpu_layer_set(oracle, problems, scratch)
        reps += 1
        elapsed = time.perf_counter() - start
        if elapsed > 10.0 or reps >= 200:
            break
    value = sum(s.algorithmic_bytes() for s in shapes) * reps / elapsed / 1e12
    return {
        "value": value,
        "unit": UNIT,
        "cores": oracle.num_threads(),
        "kind": "port",
        "sample": f"{reps} passes over one decoder layer's 4 GEMVs ({elapsed:.1f} s of host time): "
                  "C restatement of the reference's _explicit_reference_output",
        "us_per_call": elapsed * 1e6 / (reps * len(shapes)),
    }


def _sharded_layers(torch, dist, capi, device, world: int, rank: int, peak_gbs: float) -> list[dict]:
    """The two layers that are large enough to be split over the GPUs of a node (70B-style fused
    gate+up, N-split; down_proj, K-split), each with the NCCL exchange and with the exchange done
    by the GEMV kernel itself through peer memory. Per-call device time over a CUDA graph that
    cycles through several weight copies (so shards that would fit in L2 still come from HBM)."""
    from fast_kernels.dist import ShardedW4A16Linear, column_shard_packets, row_shard_packets
    from fast_kernels.workloads import SHARDED_COLUMN, SHARDED_ROW, make_problem

    lib = capi.load_library()
    results = []
    for shape, mode in ((SHARDED_COLUMN, "column"), (SHARDED_ROW, "row")):
        prob = make_problem(shape)
        q, alpha, beta = (prob[key].to(device) for key in ("q_u8", "alpha", "beta"))
        act = prob["activations"].to(device)
        stride = capi.packet_stride_bytes(128)
        packets = torch.empty(((shape.n // 128) * (shape.k // 128), stride), dtype=torch.uint8, device=device)
        capi.check(lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), packets.data_ptr(),
                                             shape.n, shape.k, 128, stride,
                                             int(torch.cuda.current_stream(device).cuda_stream)))
        shard = (column_shard_packets if mode == "column" else row_shard_packets)(
            packets, n=shape.n, k=shape.k, group_size=128, rank=rank, world=world).contiguous()
        del q, alpha, beta, packets
        copies = max(2, min(8, int(400e6 // shard.numel()) + 1))
        gen = torch.Generator().manual_seed(7)
        shards = [shard] + [shard[torch.randperm(shard.shape[0], generator=gen).to(device)].contiguous()
                            for _ in range(copies - 1)]
        for exchange in ("nccl", "peer"):
            layers = [ShardedW4A16Linear(s, n=shape.n, k=shape.k, group_size=128, mode=mode,
                                         dtype=torch.bfloat16, exchange=exchange, packets_are_local=True,
                                         max_batch=1) for s in shards]
            for layer in layers:  # eager warm-up (function attributes, communicators)
                layer(act)
            torch.cuda.synchronize(device)
            dist.barrier()
            mode_used = "cuda graph"
            try:
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream(device=device)
                side.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
                    for layer in layers:
                        layer(act)
                torch.cuda.current_stream(device).wait_stream(side)
                run = graph.replay
            except RuntimeError:
                mode_used = "eager"

                def run() -> None:
                    for layer in layers:
                        layer(act)
            for _ in range(3):
                run()
            torch.cuda.synchronize(device)
            dist.barrier()
            reps = 20
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(reps):
                run()
            stop.record()
            torch.cuda.synchronize(device)
            t = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item()) * 1e3 / (reps * len(layers))
            total_gbs = shape.algorithmic_bytes() / (us * 1e-6) / 1e9
            results.append({"layer": shape.name, "n": shape.n, "k": shape.k, "split": mode, "exchange": exchange,
                            "us_per_call": us, "aggregate_gbs": total_gbs,
                            "frac_of_n_gpu_peak": total_gbs / (peak_gbs * world), "launch": mode_used,
                            "weight_copies": len(layers)})
            del layers
        del shards, shard
        torch.cuda.empty_cache()
    return results


def run_ours(args) -> int:
    import torch
    import torch.distributed as dist
    from fast_kernels import capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the W4A16 kernels have no CPU fallback")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    layers = LayerSet(torch, capi, device)
    shapes = _layer_shapes()
    layers.launch_all()  # first launches outside capture (one-time function attributes)
    torch.cuda.synchronize(device)
    graph = layers.capture()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize(device)

    if world > 1:
        dist.barrier()
    with ClockSampler(local_rank) as clocks:
        seconds = _time_graph(torch, graph, args.steps, device)
    if world > 1:
        dist.barrier()
        t = torch.tensor([seconds], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())

    status = capi.device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: a bounded device-side wait timed out")

    step_bytes = _bytes_per_step(shapes)
    calls_per_step = len(layers.calls)
    value = step_bytes * world * args.steps / seconds / 1e12
    peak_gbs, peak_kind = _measured_peak()

    # per-shape latency: each shape's 32 distinct weight copies replayed as their own graph
    per_layer = []
    for shape in shapes:
        subset = [c for c in layers.calls if c[0].name == shape.name]
        sub_graph = layers.capture(subset)
        for _ in range(3):
            sub_graph.replay()
        reps = max(4, args.steps // 4)
        sub_seconds = _time_graph(torch, sub_graph, reps, device)
        us = sub_seconds * 1e6 / (reps * len(subset))
        gbs = shape.algorithmic_bytes() / (us * 1e-6) / 1e9
        per_layer.append({"name": shape.name, "n": shape.n, "k": shape.k, "us_per_call": us,
                          "achieved_gbs": gbs, "frac_of_peak": gbs / peak_gbs,
                          "algorithmic_bytes": shape.algorithmic_bytes()})

    e2e_steps = max(2, min(args.steps, 20))
    e2e = _e2e(torch, layers, e2e_steps, device)
    e2e_seconds = e2e["seconds"]
    if world > 1:
        t = torch.tensor([e2e_seconds], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    e2e_value = step_bytes * world * e2e_steps / e2e_seconds / 1e12

    sharded = None
    if world > 1 and not args.no_sharded:
        sharded = _sharded_layers(torch, dist, capi, device, world, rank, peak_gbs)

    if rank == 0:
        achieved_gbs = step_bytes * args.steps / seconds / 1e9  # this rank's kernels, gaps included
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": seconds * 1e3 / args.steps,
            "us_per_call": seconds * 1e6 / (args.steps * calls_per_step),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": _config(world),
            "roofline": {
                "bound": "hbm",
                "achieved": achieved_gbs,
                "peak": peak_gbs,
                "unit": "GB/s",
                "frac": achieved_gbs / peak_gbs,
                "peak_source": f"{peak_kind} (STREAM-style copy)",
                "frac_of_nominal_8tbs": achieved_gbs / 8000.0,
                "kernel": "w4a16_gemv_stream_kernel<128, 1, UnpackBF16>",
                "algorithmic_bytes_per_launch_avg": step_bytes / calls_per_step,
                # DRAM bytes per average launch: the algorithmic bytes times the ratio that one ncu
                # capture each of the largest and the smallest layer gave (dram read + write over
                # algorithmic bytes: 1.002 and 1.004; the kernel reads every packet exactly once)
                "traffic": NCU_TRAFFIC_RATIO * step_bytes / calls_per_step,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of two layer shapes "
                                  "(ratio to algorithmic bytes 1.002-1.004), scaled to the average launch",
                "per_layer": per_layer,
            },
            "e2e": {
                "value": e2e_value,
                "unit": UNIT,
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                "us_per_call": e2e_seconds * 1e6 / (e2e_steps * calls_per_step),
                "host_enqueue_us_per_call": e2e["host_seconds"] * 1e6 / (e2e_steps * calls_per_step),
                "steps": e2e_steps,
                "api": "C ABI fk_w4a16_gemv_host per call: pinned host activations in, pinned host result out",
            },
            "gpu_launches": calls_per_step * args.steps,
            "clocks": clocks.summary(),
        }
        if sharded is not None:
            line["sharded_layers"] = {
                "note": "strong scaling of single large layers over this run's GPUs (N-split + gather, "
                        "K-split + reduce); us_per_call is the max over ranks",
                "results": sharded,
            }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = _cpu_baseline_leg()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the ~10 s CPU baseline leg")
    parser.add_argument("--no-sharded", action="store_true", help="N > 1: skip the sharded-layer measurements")
    args = parser.parse_args()
    if args.impl == "reference":
        args.steps = 10 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        return run_reference_arm(args)
    args.steps = 200 if args.steps is None else args.steps
    args.warmup = 5 if args.warmup is None else args.warmup
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
