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

The timed region of K steps is repeated (`--regions`, default 15); `value` is the median region,
the spread is reported beside it. `roofline` names the kernel with the largest share of the step
and carries one entry per kernel (`kernels`) and per layer shape (`per_layer`).

`e2e` measures the same work through the C-ABI entry point that takes HOST buffers
(`fk_w4a16_gemv_host`), one call per GEMV: every call pulls its activations from pinned host
memory and stores its result to pinned host memory inside the timed region. The 128 calls of a
step are recorded once into a CUDA graph (as a decode loop would) and replayed; the eager
call-by-call figure is reported beside it.

Extra keys, measured outside the headline's timed region on one GPU: `configs` (the other
benchmark configurations: the single fp16 case, the batched sweep at 28672 x 8192, the 13B MLP at
three group sizes, the LM head), `pack` (weight packing throughput), `reference_gpu` (the
reference's own CUDA kernels, compiled unmodified into oracle/_ref, on the same layer shapes) and
`cpu_baseline`. With N > 1 -- and as a one-GPU row at N = 1 -- `sharded_layers` strong-scales the
two large sharded layers, checks every result against the fp64 oracle and reports the speed-up
over one GPU.

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
        self.pack = None
        for shape in shapes:
            prob = make_problem(shape)
            q, alpha, beta = (prob[key].to(device) for key in ("q_u8", "alpha", "beta"))
            packets = torch.empty(((shape.n // 128) * (shape.k // 128), stride), dtype=torch.uint8,
                                  device=device)

            def pack() -> None:
                capi.check(self.lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(),
                                                          packets.data_ptr(), shape.n, shape.k, 128, stride,
                                                          self.stream_ptr()))
            pack()
            if shape.name == "gate_up":
                self.pack = self._time_pack(pack, shape, q, alpha, beta, packets)
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

    def _time_pack(self, pack, shape, q, alpha, beta, packets) -> dict:
        """Throughput of the one-time weight packing on the 62 MB layer (reads q, alpha, beta;
        writes the packets), CUDA events around 5 back-to-back runs after 2 warm-ups."""
        torch = self.torch
        for _ in range(2):
            pack()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(self.device)
        start.record()
        for _ in range(5):
            pack()
        stop.record()
        torch.cuda.synchronize(self.device)
        us = start.elapsed_time(stop) * 1e3 / 5
        moved = q.numel() + 2 * alpha.numel() + 2 * beta.numel() + packets.numel()
        return {"layer": shape.name, "n": shape.n, "k": shape.k, "us_per_call": us,
                "bytes_read_plus_written": moved, "gbs": moved / (us * 1e-6) / 1e9,
                "kernel": "fk_w4a16::pack_packets_kernel<128>"}

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
        saved = self.calls
        if calls is not None:
            self.calls = calls
        try:
            return _capture(self.torch, self.device, self.launch_all)
        finally:
            self.calls = saved


def _capture(torch, device, enqueue):
    """Records `enqueue()` (which launches on the current stream) into a CUDA graph."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            enqueue()
    torch.cuda.current_stream(device).wait_stream(side)
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
    call pulls its activations from pinned host memory, runs the GEMV and delivers the result to
    pinned host memory, all inside the timed region. Measured twice: with the step's 128 calls
    recorded once into a CUDA graph and replayed, and eagerly, call by call."""
    capi = layers.capi
    lib = layers.lib
    host_in, host_out, dev_in = {}, {}, {}
    for shape, act, _, _ in layers.calls[:4]:
        host_in[shape.name] = act.cpu().pin_memory()
        host_out[shape.name] = torch.empty((1, shape.n), dtype=act.dtype).pin_memory()
        dev_in[shape.name] = torch.empty_like(act)
    h2d = sum(t.numel() * 2 for t in host_in.values()) * NUM_LAYERS
    d2h = sum(t.numel() * 2 for t in host_out.values()) * NUM_LAYERS
    plan = [(host_in[s.name].data_ptr(), packets.data_ptr(), host_out[s.name].data_ptr(),
             dev_in[s.name].data_ptr(), out.data_ptr(), s.n, s.k) for s, _, packets, out in layers.calls]
    ws, ws_bytes = layers.workspace.data_ptr(), layers.workspace.numel()

    def step() -> None:
        stream = layers.stream_ptr()
        for h_in, packets, h_out, d_in, d_out, n, k in plan:
            rc = lib.fk_w4a16_gemv_host(h_in, packets, h_out, d_in, d_out, ws, ws_bytes, 1, n, k, 128,
                                        layers.stride, capi.DTYPE_BF16, stream)
            if rc != 0:
                capi.check(rc)

    def check_results() -> None:
        # the results are real: the last call's output on the host equals the device tensor
        last_shape, _, _, last_out = layers.calls[-1]
        if not torch.equal(host_out[last_shape.name], last_out.cpu()):
            raise SystemExit("e2e: host result differs from the device result")

    step()
    torch.cuda.synchronize(device)
    # eager, call by call
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    host_begin = time.perf_counter()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    host_seconds = time.perf_counter() - host_begin  # time the host spent enqueueing
    torch.cuda.synchronize(device)
    eager_seconds = start.elapsed_time(stop) / 1e3
    check_results()
    # recorded once, replayed: what a decode loop does with a fixed sequence of calls
    for tensor in host_out.values():
        tensor.zero_()
    graph = _capture(torch, device, step)
    for _ in range(2):
        graph.replay()
    graph_seconds = _time_graph(torch, graph, steps, device)
    check_results()
    return {"seconds": graph_seconds, "eager_seconds": eager_seconds, "host_seconds": host_seconds,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}


def _chain_leg(torch, capi, layers: LayerSet, device, step_bytes: int, peak_gbs: float) -> dict:
    """The layer set through fk_w4a16_gemv_chain: each decoder layer's four GEMVs as ONE persistent
    launch (grid-wide barriers inside instead of kernel boundaries), 32 launches per step, replayed
    as a CUDA graph like the per-call step. Reported beside the per-call figure, never instead."""
    lib = layers.lib
    need = int(lib.fk_w4a16_chain_workspace_bytes(1, 128))
    workspace = torch.zeros(need, dtype=torch.uint8, device=device)
    arrays = []
    for base in range(0, len(layers.calls), 4):
        array = (capi.ChainStep * 4)()
        for slot, (shape, act, packets, out) in zip(array, layers.calls[base:base + 4]):
            slot.activations, slot.packets, slot.output = act.data_ptr(), packets.data_ptr(), out.data_ptr()
            slot.n, slot.k = shape.n, shape.k
        arrays.append(array)

    def enqueue() -> None:
        stream = layers.stream_ptr()
        for array in arrays:
            capi.check(lib.fk_w4a16_gemv_chain(array, 4, workspace.data_ptr(), workspace.numel(), 1, 128,
                                               layers.stride, capi.DTYPE_BF16, stream))

    enqueue()
    torch.cuda.synchronize(device)
    graph = _capture(torch, device, enqueue)
    for _ in range(3):
        graph.replay()
    seconds = min(_time_graph(torch, graph, 5, device) for _ in range(3)) / 5
    gbs = step_bytes / seconds / 1e9
    return {"api": "fk_w4a16_gemv_chain: 4 GEMVs per launch, 32 launches per step",
            "ms_per_step": seconds * 1e3, "us_per_layer": seconds * 1e6 / len(arrays),
            "us_per_gemv": seconds * 1e6 / len(layers.calls), "achieved_gbs": gbs, "frac_of_peak": gbs / peak_gbs,
            "kernel": "w4a16_gemv_chain_kernel<128, 1, UnpackBF16>"}


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


# ------------------------------------------------------------------------------------------
# single calls over rotated weight copies: the other configurations, the reference's kernels
# ------------------------------------------------------------------------------------------
def _rotated_copies(torch, packets, total_bytes: float = 6.0e8):
    count = max(2, int(total_bytes // packets.numel()) + 1)
    return [packets] + [packets.clone() for _ in range(count - 1)]


def _time_rotation(torch, device, enqueue_one, copies, reps: int = 5) -> float:
    """Microseconds per call: one CUDA graph that calls `enqueue_one(copy)` once per weight copy
    (the copies together exceed L2 several times over), best of `reps` replays after 2 warm-ups."""
    enqueue_one(copies[0])
    torch.cuda.synchronize(device)

    def all_copies() -> None:
        for copy in copies:
            enqueue_one(copy)

    graph = _capture(torch, device, all_copies)
    for _ in range(2):
        graph.replay()
    best = min(_time_graph(torch, graph, 1, device) for _ in range(reps))
    return best * 1e6 / len(copies)


def _configs_leg(torch, capi, device, peak_gbs: float) -> list[dict]:
    """Per-call device time of the benchmark configurations the headline does not cover."""
    from fast_kernels.workloads import EDGE_SHAPES, REFERENCE_CASE, LayerShape, make_problem

    lib = capi.load_library()
    results = []

    def packed(shape, seed=None):
        prob = make_problem(shape, seed=seed)
        q, alpha, beta = (prob[key].to(device) for key in ("q_u8", "alpha", "beta"))
        stride = capi.packet_stride_bytes(shape.group_size)
        packets = torch.empty(((shape.n // 128) * (shape.k // shape.group_size), stride), dtype=torch.uint8,
                              device=device)
        capi.check(lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), packets.data_ptr(),
                                             shape.n, shape.k, shape.group_size, stride,
                                             int(torch.cuda.current_stream(device).cuda_stream)))
        torch.cuda.synchronize(device)
        return prob, packets

    def measure(config: str, shape, act, copies, workspace) -> None:
        code = capi.DTYPE_BF16 if shape.dtype == "bf16" else capi.DTYPE_F16
        out = torch.empty((shape.batch, shape.n), dtype=act.dtype, device=device)
        stride = capi.packet_stride_bytes(shape.group_size)

        def one(copy) -> None:
            capi.check(lib.fk_w4a16_gemv(act.data_ptr(), copy.data_ptr(), out.data_ptr(), workspace.data_ptr(),
                                         workspace.numel(), shape.batch, shape.n, shape.k, shape.group_size,
                                         stride, code, int(torch.cuda.current_stream(device).cuda_stream)))

        us = _time_rotation(torch, device, one, copies)
        gbs = shape.algorithmic_bytes() / (us * 1e-6) / 1e9
        results.append({"config": config, "name": shape.name, "batch": shape.batch, "n": shape.n, "k": shape.k,
                        "group_size": shape.group_size, "dtype": shape.dtype, "us_per_call": us,
                        "achieved_gbs": gbs, "frac_of_peak": gbs / peak_gbs,
                        "algorithmic_bytes": shape.algorithmic_bytes(),
                        "kernel": capi.describe_plan(shape.batch, shape.n, shape.k, shape.group_size, code),
                        "weight_copies": len(copies)})

    def workspace_for(shape):
        need = int(lib.fk_w4a16_workspace_bytes(shape.batch, shape.n, shape.k, shape.group_size))
        return torch.zeros(need, dtype=torch.uint8, device=device)

    # configs[0]: the single fp16 case, seed 0
    prob, packets = packed(REFERENCE_CASE, seed=0)
    measure("configs[0]", REFERENCE_CASE, prob["activations"].to(device), _rotated_copies(torch, packets),
            workspace_for(REFERENCE_CASE))
    # configs[2]: batched sweep over one set of weights (per-group uint4 zero points)
    base = LayerShape("mlp_up", 28672, 8192, zero_point=None)
    prob, packets = packed(base)
    copies = _rotated_copies(torch, packets)
    gen = torch.Generator().manual_seed(2)
    for batch in (1, 2, 4, 8, 16):
        shape = LayerShape(f"mlp_up_m{batch}", 28672, 8192, batch=batch, zero_point=None)
        act = torch.randn((batch, shape.k), generator=gen).to(torch.bfloat16).to(device)
        measure("configs[2]", shape, act, copies, workspace_for(shape))
    del copies, packets
    torch.cuda.empty_cache()
    # configs[4]: 13B MLP at three group sizes (fp16, asymmetric zeros), and the LM head
    for shape in EDGE_SHAPES:
        prob, packets = packed(shape)
        measure("configs[4]", shape, prob["activations"].to(device), _rotated_copies(torch, packets, 8.0e8),
                workspace_for(shape))
        del packets
        torch.cuda.empty_cache()
    return results


def _reference_gpu_leg(torch, capi, device) -> dict:
    """The reference's own CUDA kernels (arc_w4a16.cu compiled unmodified into oracle/_ref) on the
    four layer shapes -- fp16, group 128, the only type it has -- timed the same way as `configs`:
    its scalar path as its Python op chains it (group-sum prepass + arc_w4a16_forward) and its
    vendor subject (packet dequant + cuBLASLt). Baseline only; never on the product path."""
    from fast_kernels.workloads import LayerShape, make_problem
    from oracle import reference_gpu as ref

    if not ref.available():
        return {"unavailable": "oracle/_ref/libfk_reference.so is not built (no reference checkout at build time)"}
    lib = capi.load_library()
    rows = []
    for base in _layer_shapes():
        shape = LayerShape(base.name, base.n, base.k, dtype="fp16")
        prob = make_problem(shape)
        q, alpha, beta, act = (prob[key].to(device) for key in ("q_u8", "alpha", "beta", "activations"))
        packets = torch.empty(((shape.n // 128) * (shape.k // 128), 8704), dtype=torch.uint8, device=device)
        capi.check(lib.fk_w4a16_pack_packets(q.data_ptr(), alpha.data_ptr(), beta.data_ptr(), packets.data_ptr(),
                                             shape.n, shape.k, 128, 8704, 0))
        torch.cuda.synchronize(device)
        copies = _rotated_copies(torch, packets, 3.0e8)
        sums = torch.empty((1, shape.k // 128), dtype=torch.float32, device=device)
        out = torch.empty((1, shape.n), dtype=torch.float16, device=device)
        weight = torch.empty((shape.n, shape.k), dtype=torch.float16, device=device)
        lt_ws = torch.empty(32 << 20, dtype=torch.uint8, device=device)

        def scalar(copy) -> None:
            stream = int(torch.cuda.current_stream(device).cuda_stream)
            ref.group_sums(act.data_ptr(), sums.data_ptr(), 1, shape.k, 128, stream)
            ref.forward(act.data_ptr(), copy.data_ptr(), sums.data_ptr(), out.data_ptr(), 1, shape.n, shape.k, 128,
                        stream)

        def vendor(copy) -> None:
            stream = int(torch.cuda.current_stream(device).cuda_stream)
            ref.cublaslt_after_packet_dequant(act.data_ptr(), copy.data_ptr(), out.data_ptr(), weight.data_ptr(),
                                              lt_ws.data_ptr(), lt_ws.numel(), 1, shape.n, shape.k, 128, stream)

        ws = torch.zeros(int(lib.fk_w4a16_workspace_bytes(1, shape.n, shape.k, 128)), dtype=torch.uint8,
                         device=device)

        def ours(copy) -> None:
            capi.check(lib.fk_w4a16_gemv(act.data_ptr(), copy.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                                         1, shape.n, shape.k, 128, 8704, capi.DTYPE_F16,
                                         int(torch.cuda.current_stream(device).cuda_stream)))

        row = {"name": shape.name, "n": shape.n, "k": shape.k, "dtype": "fp16", "group_size": 128}
        row["reference_scalar_us"] = _time_rotation(torch, device, scalar, copies, reps=3)
        try:
            row["reference_cublaslt_after_packet_dequant_us"] = _time_rotation(torch, device, vendor, copies, reps=3)
        except Exception as exc:  # cuBLASLt under capture is the reference's affair, not ours
            row["reference_cublaslt_after_packet_dequant_us"] = None
            row["cublaslt_note"] = f"{type(exc).__name__}: {exc}"[:160]
        row["this_library_fp16_us"] = _time_rotation(torch, device, ours, copies, reps=3)
        rows.append(row)
        del copies, packets, weight
        torch.cuda.empty_cache()
    return {"note": "reference kernels: csrc/kernels/decode_quant_linear/arc_w4a16.cu of the reference, "
                    "compiled for sm_100a without changes; us per call, CUDA graph over rotated weight copies",
            "layers": rows}


# ------------------------------------------------------------------------------------------
# sharded layers
# ------------------------------------------------------------------------------------------
def _sharded_layers(torch, dist, capi, device, world: int, rank: int, peak_gbs: float) -> list[dict]:
    """The two layers that are large enough to be split over the GPUs of a node (70B-style fused
    gate+up, N-split; down_proj, K-split): first on ONE GPU (every rank times the whole layer on
    its own device; rank 0's figure is the strong-scaling baseline), then sharded, with the NCCL
    exchange and with the exchange done by the GEMV kernel itself through peer memory. Every
    sharded result is checked against the fp64 oracle on a 512-column slice and must be bit-equal
    on all ranks. Per-call device time over a CUDA graph that cycles through several weight copies
    (so shards that would fit in L2 still come from HBM), maximum over ranks."""
    from fast_kernels.workloads import SHARDED_COLUMN, SHARDED_ROW, make_problem
    from oracle import w4a16_oracle as oracle

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
        torch.cuda.synchronize(device)
        del q, alpha, beta
        cols = slice(shape.n // 2 - 256, shape.n // 2 + 256)  # straddles a shard boundary at every world size
        y64 = oracle.gemv_f64(oracle.bits_of(prob["activations"]), prob["q_u8"][cols].numpy(),
                              oracle.bits_of(prob["alpha"][cols]), oracle.bits_of(prob["beta"][cols]), 128,
                              oracle.BF16)

        # ---- one GPU: the whole layer through fk_w4a16_gemv -------------------------------------
        copies = _rotated_copies(torch, packets, 5.0e8)
        ws = torch.zeros(int(lib.fk_w4a16_workspace_bytes(1, shape.n, shape.k, 128)), dtype=torch.uint8,
                         device=device)
        out1 = torch.empty((1, shape.n), dtype=torch.bfloat16, device=device)

        def whole(copy) -> None:
            capi.check(lib.fk_w4a16_gemv(act.data_ptr(), copy.data_ptr(), out1.data_ptr(), ws.data_ptr(), ws.numel(),
                                         1, shape.n, shape.k, 128, stride, capi.DTYPE_BF16,
                                         int(torch.cuda.current_stream(device).cuda_stream)))

        one_gpu_us = _time_rotation(torch, device, whole, copies)
        whole(copies[0])
        torch.cuda.synchronize(device)
        err1 = oracle.max_rel_err(out1[:, cols].float().cpu().numpy(), y64)
        if world > 1:
            t = torch.tensor([one_gpu_us], dtype=torch.float64, device=device)
            dist.broadcast(t, src=0)
            one_gpu_us = float(t.item())
        gbs1 = shape.algorithmic_bytes() / (one_gpu_us * 1e-6) / 1e9
        results.append({"layer": shape.name, "n": shape.n, "k": shape.k, "split": "none", "exchange": "none",
                        "gpus": 1, "us_per_call": one_gpu_us, "aggregate_gbs": gbs1,
                        "frac_of_n_gpu_peak": gbs1 / peak_gbs, "max_rel_err": err1, "speedup_vs_1gpu": 1.0,
                        "launch": "cuda graph", "weight_copies": len(copies)})
        if err1 > 1e-2:
            results[-1]["failed"] = f"max_rel_err {err1:.3e}"
        del copies, ws
        torch.cuda.empty_cache()
        if world == 1:
            del packets
            continue

        # ---- sharded over the run's GPUs ----------------------------------------------------------
        from fast_kernels.dist import ShardedW4A16Linear, column_shard_packets, row_shard_packets

        shard = (column_shard_packets if mode == "column" else row_shard_packets)(
            packets, n=shape.n, k=shape.k, group_size=128, rank=rank, world=world).contiguous().clone()
        del packets
        torch.cuda.empty_cache()
        count = max(2, min(8, int(400e6 // shard.numel()) + 1))
        shards = [shard] + [shard.clone() for _ in range(count - 1)]
        for exchange in ("nccl", "peer"):
            layers = [ShardedW4A16Linear(s, n=shape.n, k=shape.k, group_size=128, mode=mode,
                                         dtype=torch.bfloat16, exchange=exchange, packets_are_local=True,
                                         max_batch=1) for s in shards]
            result = None
            for layer in layers:  # eager warm-up (function attributes, communicators)
                result = layer(act)
            torch.cuda.synchronize(device)
            # every layer object holds the same weights: check the last one's result
            got = result[:, cols].float().cpu().numpy()
            err = oracle.max_rel_err(got, y64)
            bits = result.view(torch.int16).to(torch.int64)
            checksum = torch.stack([bits.sum(), (bits * torch.arange(1, bits.numel() + 1, device=device)).sum()])
            gathered = [torch.empty_like(checksum) for _ in range(world)]
            dist.all_gather(gathered, checksum)
            ranks_agree = all(torch.equal(g, checksum) for g in gathered)
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
                            "gpus": world, "us_per_call": us, "aggregate_gbs": total_gbs,
                            "frac_of_n_gpu_peak": total_gbs / (peak_gbs * world), "max_rel_err": err,
                            "ranks_bit_equal": ranks_agree, "speedup_vs_1gpu": one_gpu_us / us,
                            "launch": mode_used, "weight_copies": len(layers)})
            status = capi.device_status()
            if err > 1e-2 or not ranks_agree or status != 0:
                # recorded in the line (which is still printed); the run then exits non-zero
                results[-1]["failed"] = (f"max_rel_err {err:.3e}, ranks bit-equal {ranks_agree}, "
                                         f"device status {status}")
            del layers
        del shards, shard
        torch.cuda.empty_cache()
    return results


# ------------------------------------------------------------------------------------------
# the other half of a decode step: paged-KV attention (the reference's clustered_page_decode suite)
# ------------------------------------------------------------------------------------------
PAGE_DECODE_SHAPES = [
    # benchmarks/suites/clustered_page_decode.toml of the reference: name, batch, page, max_len, q, kv, dim
    ("gqa4_short_page16", 4, 16, 256, 32, 8, 128),
    ("gqa4_long_page16", 4, 16, 2048, 32, 8, 128),
    ("mqa8_long_page32", 2, 32, 4096, 32, 4, 128),
    ("mqa32_long_page32", 2, 32, 4096, 32, 1, 128),
    ("gqa2_short_page32_h64", 8, 32, 512, 16, 8, 64),
    # a serving-sized batch: 32 requests of up to 4096 tokens, Llama-3-8B heads (537 MB of bf16 pages)
    ("gqa4_batch32_4k_page16", 32, 16, 4096, 32, 8, 128),
]


def _page_decode_leg(torch, device, peak_gbs: float) -> dict:
    """Per-call device time of the paged-KV decode attention through the C ABI
    (fk_page_decode_forward) on the shapes of the reference's suite, every page format, page tables
    fragmented by a seeded permutation; the page copies of one CUDA graph together exceed L2 several
    times. Each result is checked against the fp64 oracle on request 0. Where the reference's own
    kernels are built (oracle/_ref), their time on the same inputs stands beside it."""
    import ctypes
    import importlib

    import numpy as np
    from fast_kernels import page_decode_capi as pdc
    from oracle import page_decode_oracle as pd_oracle
    from oracle import reference_page_decode_gpu as refgpu

    ops = importlib.import_module("fast_kernels.ops.clustered_page_decode")
    lib = pdc.load_library()
    rows = []

    def stream() -> int:  # the capturing stream while a graph is recorded
        return int(torch.cuda.current_stream(device).cuda_stream)

    for name, batch, page, max_len, q_heads, kv_heads, dim in PAGE_DECODE_SHAPES:
        generator = torch.Generator().manual_seed(batch + max_len)
        lens = torch.randint(max(page, max_len - page + 1), max_len + 1, (batch,), generator=generator, dtype=torch.int32)
        query = torch.randn((batch, q_heads, dim), generator=generator).to(torch.bfloat16).to(device)
        torch.manual_seed(batch * max_len)
        keys = torch.randn((batch, kv_heads, max_len, dim), device=device).to(torch.bfloat16)
        values = torch.randn((batch, kv_heads, max_len, dim), device=device).to(torch.bfloat16)
        tokens = int(lens.sum())
        for label in ("bf16_kv", "bf16_kv_rotated", "fp8_kv", "fp8_kv_rotated", "int8_kv", "int8_kv_rotated"):
            # "*_rotated": keys stored with their rotary embedding applied, as serving engines keep
            # them; the kernel then rotates the query only (and runs on the tensor cores)
            layout, rotated = label.replace("_rotated", ""), label.endswith("_rotated")
            if layout != "bf16_kv" and not rotated and batch >= 32:
                continue  # the large batch: 8-bit pages in the form serving engines store only
            build = {"bf16_kv": ops.pack_paged_kv_bf16, "fp8_kv": ops.quantize_paged_kv_fp8,
                     "int8_kv": ops.quantize_paged_kv_int8}[layout]
            cache = build(keys, values, lens, page_size=page, fragment_pages=True, seed=1,
                          key_rope_theta=10000.0 if rotated else None)
            plan = ops.plan_clustered_page_decode(page_table=cache.page_table, seq_lens=cache.seq_lens,
                                                  num_q_heads=q_heads, num_kv_heads=kv_heads, head_dim=dim,
                                                  page_size=page, kv_layout=layout, use_cache=False)
            descriptors = plan.device_tensors(device)
            element = 2 if layout == "bf16_kv" else 1
            algorithmic = tokens * kv_heads * dim * 2 * element + 2 * query.numel() * 2
            if element == 1:
                algorithmic += tokens * kv_heads * (dim // 64) * 4 + cache.total_pages * kv_heads * (dim // 64) * 4
            key_copies = _rotated_copies(torch, cache.key_pages.view(torch.uint8).reshape(-1), 3.0e8)
            value_copies = _rotated_copies(torch, cache.value_pages.view(torch.uint8).reshape(-1), 3.0e8)
            workspace = torch.zeros(int(lib.fk_page_decode_workspace_bytes(batch, q_heads, kv_heads, dim)),
                                    dtype=torch.uint8, device=device)
            out = torch.empty_like(query)

            def arguments(copy: int):
                a = pdc.PageDecodeArgs()
                a.query, a.output = query.data_ptr(), out.data_ptr()
                a.key_pages, a.value_pages = key_copies[copy].data_ptr(), value_copies[copy].data_ptr()
                a.key_scales = 0 if cache.key_scales is None else cache.key_scales.data_ptr()
                a.value_scales = 0 if cache.value_scales is None else cache.value_scales.data_ptr()
                for field in ("run_base_pages", "run_page_counts", "run_logical_starts", "run_last_page_lens",
                              "request_run_offsets", "seq_lens"):
                    setattr(a, field, descriptors[field].data_ptr())
                a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
                a.batch, a.num_runs, a.num_q_heads, a.num_kv_heads = batch, plan.num_runs, q_heads, kv_heads
                a.head_dim, a.page_size, a.kv_format = dim, page, ops.KV_FORMAT_IDS[layout]
                a.keys_are_rotated = int(rotated)
                a.max_pages_hint, a.softmax_scale, a.rope_theta = plan.max_pages, 1.0 / dim**0.5, 10000.0
                a.stream = stream()
                a.flags = pdc.FLAG_EARLY_DESCRIPTORS  # the descriptors are uploaded once, nothing on the device writes them
                return a

            def ours(copy: int) -> None:
                pdc.check(lib.fk_page_decode_forward(ctypes.byref(arguments(copy))))

            us = _time_rotation(torch, device, ours, list(range(len(key_copies))))
            info = pdc.describe_plan(arguments(0))
            # request 0 against the fp64 oracle (same bytes; bound: 2e-3 + 8e-3 |y|)
            first = slice(int(plan.request_run_offsets_cpu[0]), int(plan.request_run_offsets_cpu[1]))

            def raw(t):
                return (t.view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16
                        else t.view(torch.uint8).cpu().numpy())

            want = pd_oracle.page_decode_f64(
                raw(query[:1]), raw(cache.key_pages), raw(cache.value_pages),
                None if cache.key_scales is None else cache.key_scales.cpu().numpy(),
                None if cache.value_scales is None else cache.value_scales.cpu().numpy(),
                plan.run_base_pages_cpu.numpy()[first], plan.run_page_counts_cpu.numpy()[first],
                plan.run_logical_starts_cpu.numpy()[first], plan.run_last_page_lens_cpu.numpy()[first],
                np.asarray([0, first.stop - first.start]), lens.numpy()[:1], kv_format=ops.KV_FORMAT_IDS[layout],
                keys_are_rotated=rotated, softmax_scale=1.0 / dim**0.5, rope_theta=10000.0)
            pdc.check(lib.fk_page_decode_forward(ctypes.byref(arguments(0))))
            torch.cuda.synchronize(device)
            worst, scaled = pd_oracle.max_abs_and_scaled_error(out[:1].float().cpu().numpy().astype(np.float64), want,
                                                               2e-3, 8e-3)
            row = {"shape": name, "layout": label, "kernel": info["kernel"], "batch": batch, "tokens": tokens,
                   "us_per_call": us,
                   "algorithmic_bytes": algorithmic, "gbs": algorithmic / us / 1e3,
                   "frac": algorithmic / us / 1e3 / peak_gbs, "blocks": int(info["blocks"]),
                   "splits": int(info["splits"]), "warps": int(info["warps"]), "max_abs_err": worst,
                   "error_over_bound": scaled, "page_copies": len(key_copies)}
            if scaled > 1.0:
                row["failed"] = "result is off the fp64 oracle"
            if refgpu.available() and layout == "bf16_kv" and batch < 32:
                rotated_flag = int(rotated)
                group = q_heads // kv_heads
                modes = [("reference_cluster_us", 1, max(1, plan.cluster_size))]
                if group <= 8:
                    modes.append(("reference_direct_us", 0, 1))
                for key, clustered, cluster_size in modes:
                    def theirs(copy: int) -> None:
                        refgpu.forward(query=query, key_pages=key_copies[copy], value_pages=value_copies[copy],
                                       key_scales=cache.key_scales, value_scales=cache.value_scales,
                                       runs=descriptors, seq_lens=descriptors["seq_lens"], output=out, batch=batch,
                                       num_q_heads=q_heads, num_kv_heads=kv_heads, head_dim=dim, page_size=page,
                                       group_tile=plan.group_tile, use_clustered_kernel=clustered,
                                       cluster_size=cluster_size, kv_format=0, keys_are_rotated=bool(rotated_flag),
                                       softmax_scale=1.0 / dim**0.5, rope_theta=10000.0, stream=stream())

                    row[key] = _time_rotation(torch, device, theirs, list(range(min(8, len(key_copies)))), reps=2)
            rows.append(row)
            del key_copies, value_copies
    if pdc.device_status() != 0:
        rows.append({"failed": "device status word set: a bounded wait timed out"})
    return {"note": "paged-KV decode attention (fk_page_decode_forward), device time per call, page copies "
                    "rotated so that every call reads HBM; frac is of the measured HBM peak; calls follow one "
                    "another in one stream under programmatic dependent launch with "
                    "FK_PAGE_DECODE_FLAG_EARLY_DESCRIPTORS (the descriptors are static)",
            "results": rows}



def _kernel_table(capi, per_layer: list[dict], ms_per_step: float) -> list[dict]:
    """Per kernel (template instantiation): launches per step, time share and achieved bandwidth,
    from the per-shape timings."""
    table: dict[str, dict] = {}
    for row in per_layer:
        name = capi.describe_plan(1, row["n"], row["k"], 128, capi.DTYPE_BF16).split(" grid=")[0]
        entry = table.setdefault(name, {"name": name, "launches_per_step": 0, "us_per_step": 0.0,
                                        "bytes_per_step": 0, "layers": []})
        entry["launches_per_step"] += NUM_LAYERS
        entry["us_per_step"] += NUM_LAYERS * row["us_per_call"]
        entry["bytes_per_step"] += NUM_LAYERS * row["algorithmic_bytes"]
        entry["layers"].append(row["name"])
    peak_gbs, _ = _measured_peak()
    out = []
    for entry in table.values():
        us_per_call = entry["us_per_step"] / entry["launches_per_step"]
        achieved = entry["bytes_per_step"] / (entry["us_per_step"] * 1e-6) / 1e9
        out.append({"name": entry["name"], "layers": entry["layers"],
                    "launches_per_step": entry["launches_per_step"], "us_per_call": us_per_call,
                    "algorithmic_bytes_per_launch": entry["bytes_per_step"] / entry["launches_per_step"],
                    "share_of_step": entry["us_per_step"] / (ms_per_step * 1e3),
                    "achieved": achieved, "frac": achieved / peak_gbs})
    return sorted(out, key=lambda e: -e["share_of_step"])


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

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize(device)

    # R timed regions of exactly `steps` steps each; the headline is the median region
    regions = []
    with ClockSampler(local_rank) as clocks:
        for _ in range(max(1, args.regions)):
            if world > 1:
                dist.barrier()
            seconds = _time_graph(torch, graph, args.steps, device)
            if world > 1:
                dist.barrier()
                t = torch.tensor([seconds], dtype=torch.float64, device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                seconds = float(t.item())
            regions.append(seconds)
    seconds = statistics.median(regions)

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
        sub_seconds = min(_time_graph(torch, sub_graph, reps, device) for _ in range(3))
        us = sub_seconds * 1e6 / (reps * len(subset))
        gbs = shape.algorithmic_bytes() / (us * 1e-6) / 1e9
        per_layer.append({"name": shape.name, "n": shape.n, "k": shape.k, "us_per_call": us,
                          "achieved_gbs": gbs, "frac_of_peak": gbs / peak_gbs,
                          "algorithmic_bytes": shape.algorithmic_bytes(),
                          "kernel": capi.describe_plan(1, shape.n, shape.k, 128, capi.DTYPE_BF16)})

    # the same step as 32 chains of 4 GEMVs each (one persistent launch per decoder layer)
    chain = _chain_leg(torch, capi, layers, device, step_bytes, peak_gbs)

    e2e_steps = max(2, min(args.steps, 20))
    e2e = _e2e(torch, layers, e2e_steps, device)
    e2e_seconds = e2e["seconds"]
    if world > 1:
        t = torch.tensor([e2e_seconds], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    e2e_value = step_bytes * world * e2e_steps / e2e_seconds / 1e12

    pack = layers.pack
    del graph, layers
    torch.cuda.empty_cache()

    sharded = None
    sharded_error = None
    if not args.no_sharded:
        try:
            sharded = _sharded_layers(torch, dist, capi, device, world, rank, peak_gbs)
        except Exception as exc:  # the headline above is measured already: report, do not lose it
            sharded_error = f"{type(exc).__name__}: {exc}"[:300]

    extra = {}
    if world == 1 and not args.no_extras:
        extra["configs"] = _configs_leg(torch, capi, device, peak_gbs)
        extra["reference_gpu"] = _reference_gpu_leg(torch, capi, device)
        try:
            extra["page_decode"] = _page_decode_leg(torch, device, peak_gbs)
        except Exception as exc:  # the headline above is measured already: report, do not lose it
            extra["page_decode"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0:
        ms_per_step = seconds * 1e3 / args.steps
        step_gbs = step_bytes * args.steps / seconds / 1e9  # this rank's kernels, gaps included
        kernels = _kernel_table(capi, per_layer, ms_per_step)
        top = kernels[0]
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "us_per_call": seconds * 1e6 / (args.steps * calls_per_step),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": _config(world),
            "regions": {
                "count": len(regions),
                "steps_each": args.steps,
                "ms_per_step_median": ms_per_step,
                "ms_per_step_min": min(regions) * 1e3 / args.steps,
                "ms_per_step_max": max(regions) * 1e3 / args.steps,
                "value_min": step_bytes * world * args.steps / max(regions) / 1e12,
                "value_max": step_bytes * world * args.steps / min(regions) / 1e12,
            },
            "roofline": {
                "bound": "hbm",
                # the kernel with the largest share of the step: its algorithmic bytes per launch
                # over its average launch duration inside its own back-to-back graph
                "kernel": top["name"],
                "achieved": top["achieved"],
                "peak": peak_gbs,
                "unit": "GB/s",
                "frac": top["frac"],
                "peak_source": f"{peak_kind} (STREAM-style copy)",
                "frac_of_nominal_8tbs": top["achieved"] / 8000.0,
                "algorithmic_bytes_per_launch": top["algorithmic_bytes_per_launch"],
                # DRAM bytes per launch: the algorithmic bytes times the ratio that one ncu capture
                # each of the largest and the smallest layer gave (dram read + write over
                # algorithmic bytes: 1.002 and 1.004; the kernels read every packet exactly once)
                "traffic": NCU_TRAFFIC_RATIO * top["algorithmic_bytes_per_launch"],
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of two layer shapes "
                                  "(ratio to algorithmic bytes 1.002-1.004), scaled to this kernel's average launch",
                "step": {"achieved": step_gbs, "frac": step_gbs / peak_gbs,
                         "frac_of_nominal_8tbs": step_gbs / 8000.0,
                         "algorithmic_bytes_per_launch_avg": step_bytes / calls_per_step,
                         "note": "whole step, gaps between launches included"},
                "kernels": kernels,
                "per_layer": per_layer,
            },
            "e2e": {
                "value": e2e_value,
                "unit": UNIT,
                "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
                "us_per_call": e2e_seconds * 1e6 / (e2e_steps * calls_per_step),
                "steps": e2e_steps,
                "api": "C ABI fk_w4a16_gemv_host per GEMV (pinned host activations in, pinned host result out); "
                       "the step's 128 calls recorded once into a CUDA graph and replayed",
                "eager": {
                    "value": step_bytes * e2e_steps / e2e["eager_seconds"] / 1e12,
                    "us_per_call": e2e["eager_seconds"] * 1e6 / (e2e_steps * calls_per_step),
                    "host_enqueue_us_per_call": e2e["host_seconds"] * 1e6 / (e2e_steps * calls_per_step),
                    "note": "the same calls issued one by one from Python (ctypes), this rank",
                },
            },
            "gpu_launches": calls_per_step * args.steps,
            "clocks": clocks.summary(),
            "pack": pack,
            "layer_chain": chain,
        }
        if sharded_error is not None:
            line["sharded_layers"] = {"error": sharded_error}
        if sharded is not None:
            line["sharded_layers"] = {
                "note": "strong scaling of single large layers over this run's GPUs (N-split + gather, "
                        "K-split + reduce) against the same layer on one GPU; us_per_call is the max over ranks; "
                        "max_rel_err is against the fp64 oracle on a 512-column slice",
                "results": sharded,
            }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = _cpu_baseline_leg()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if sharded_error is not None:
        print(f"sharded_layers: {sharded_error}", file=sys.stderr)
        return 1
    if sharded is not None and any("failed" in row for row in sharded):
        print("sharded_layers: a result failed its check (see the 'failed' fields)", file=sys.stderr)
        return 1
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--regions", type=int, default=15, help="timed regions of --steps steps each")
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the ~10 s CPU baseline leg")
    parser.add_argument("--no-sharded", action="store_true", help="skip the sharded-layer measurements")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the other configurations and the reference's GPU kernels")
    args = parser.parse_args()
    if args.impl == "reference":
        args.steps = 10 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        return run_reference_arm(args)
    args.steps = 100 if args.steps is None else args.steps
    args.warmup = 5 if args.warmup is None else args.warmup
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
