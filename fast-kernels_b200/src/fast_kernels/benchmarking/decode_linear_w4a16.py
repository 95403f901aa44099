"""Runner for suites of the ``decode_quant_linear`` family (what ``fk bench`` executes).

Follows the flow of the reference's runner (src/fast_kernels/benchmarking/decode_linear_w4a16.py
:292-682): per dtype x layout x shape it draws seeded inputs, packs them, gates every subject on
agreement with an explicit fp32 torch expression under the suite's tolerances, then times the two
baselines (``baselines.ids[0]`` = torch reference, ``[1]`` = vendor GEMM, by position) and every
kernel id. Differences: device time comes from CUDA events and is what ``latency_us_*`` reports
(the wall clock, 4 warm-up + 12 timed calls as in the reference, is kept beside it) and is taken over CUDA-graph replays; weights rotate
over enough copies to exceed L2 so the figures are HBM figures; ``metrics`` carries the achieved
bandwidth. Without a GPU every case is emitted as ``skipped`` with the reason.
"""

from __future__ import annotations

from statistics import median
from time import perf_counter
from typing import Any, Callable

from fast_kernels.registry import kernel_registry
from fast_kernels.schemas import BenchmarkCase, BenchmarkSuite, ShapeCase

WARMUP_ITERS = 4
TIMING_ITERS = 12
ROTATION_BYTES = 512 * 1024 * 1024  # distinct weight bytes cycled through, > 4x the L2
DEFAULT_HBM_PEAK_GBS = 6542.7       # measured copy bandwidth of the B200 this was tuned on


def _seed_for_case(batch: int, n: int, k: int, group_size: int) -> int:
    # the reference's rule (:148-149), so that both builds draw the same case
    return (batch * 1_000_003 + n * 1009 + k * 101 + group_size) % (2**31 - 1)


def _p95(samples: list[float]) -> float:
    ordered = sorted(samples)
    return ordered[min(len(ordered) - 1, int(round(0.95 * (len(ordered) - 1))))]


def _make_inputs(torch: Any, suite: BenchmarkSuite, shape: ShapeCase, group: int, dtype: Any, device: Any):
    """Seeded on the CPU generator, then moved. Distribution knobs come from ``[metadata]``:
    activation_scale (default 0.25), scale_range (default [0.02, 0.2]), zero_point (default
    "uniform" = uint4 per group; an integer pins it) -- defaults are the reference's recipe."""
    meta = suite.metadata
    n, k, batch = shape.require_dimension("n"), shape.require_dimension("k"), shape.batch
    gen = torch.Generator().manual_seed(int(meta.get("seed", _seed_for_case(batch, n, k, group))))
    groups = k // group
    lo, hi = meta.get("scale_range", [0.02, 0.2])
    act = (float(meta.get("activation_scale", 0.25)) * torch.randn((batch, k), generator=gen)).to(dtype)
    q_u8 = torch.randint(0, 256, (n, k // 2), generator=gen, dtype=torch.uint8)
    alpha = (lo + (hi - lo) * torch.rand((n, groups), generator=gen)).to(dtype)
    zero = meta.get("zero_point", "uniform")
    if zero == "uniform":
        zp = torch.randint(0, 16, (n, groups), generator=gen, dtype=torch.int16).to(dtype)
    else:
        zp = torch.full((n, groups), float(zero), dtype=dtype)
    beta = -(alpha * zp)
    return tuple(t.contiguous().to(device) for t in (act, q_u8, alpha, beta))


def _explicit_reference(torch: Any, act: Any, q_u8: Any, alpha: Any, beta: Any, group: int) -> Any:
    low = (q_u8 & 0x0F).to(torch.float32)
    high = (q_u8 >> 4).to(torch.float32)
    q = torch.stack((low, high), dim=-1).reshape(q_u8.shape[0], q_u8.shape[1] * 2)
    weight = alpha.float().repeat_interleave(group, dim=1) * q + beta.float().repeat_interleave(group, dim=1)
    return (act.float() @ weight.t()).to(act.dtype)


_CAPTURE_STREAMS: dict[int, Any] = {}


def _capture_stream(torch: Any) -> Any:
    """One capturing stream per device for the whole run: the ops keep a scratch buffer per
    (device, stream), so a fresh stream per measurement would leave one buffer behind each time."""
    device = torch.cuda.current_device()
    if device not in _CAPTURE_STREAMS:
        _CAPTURE_STREAMS[device] = torch.cuda.Stream()
    return _CAPTURE_STREAMS[device]


def _time_device(torch: Any, calls: list[Callable[[], Any]], iters: int) -> list[float]:
    """Device time per call in microseconds, one sample per replay of a CUDA graph that holds one
    launch per entry of ``calls`` (distinct weight copies), so that host launch overhead is not in
    the figure. Falls back to one event pair per eager call if capture is refused."""
    for fn in calls[: max(1, min(len(calls), WARMUP_ITERS))]:
        fn()
    torch.cuda.synchronize()
    try:
        graph = torch.cuda.CUDAGraph()
        side = _capture_stream(torch)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            # the ops keep their scratch per (device, stream) and allocate it on a stream's first
            # call, which must not happen under capture: make that call on the capturing stream
            calls[0]()
        side.synchronize()
        with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
            for fn in calls:
                fn()
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        samples = []
        for _ in range(iters):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            samples.append(start.elapsed_time(stop) * 1e3 / len(calls))
        return samples
    except RuntimeError:
        torch.cuda.synchronize()
    pairs = []
    for i in range(iters):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        calls[i % len(calls)]()
        stop.record()
        pairs.append((start, stop))
    torch.cuda.synchronize()
    return [a.elapsed_time(b) * 1e3 for a, b in pairs]


def _time_wall(torch: Any, calls: list[Callable[[], Any]]) -> list[float]:
    samples = []
    for i in range(WARMUP_ITERS + TIMING_ITERS):
        begin = perf_counter()
        calls[i % len(calls)]()
        torch.cuda.synchronize()
        if i >= WARMUP_ITERS:
            samples.append((perf_counter() - begin) * 1e6)
    return samples


def _skipped(suite: BenchmarkSuite, reason: str) -> list[BenchmarkCase]:
    from fast_kernels.benchmarking import case_id

    cases = []
    for kind, ids in (("kernel", suite.kernels.ids), ("baseline", suite.baselines.ids)):
        for subject in ids:
            for dtype in suite.dtypes:
                for layout in suite.layouts:
                    for shape in suite.shapes:
                        cases.append(BenchmarkCase(
                            case_id=case_id(kind, subject, dtype, layout, shape.name), subject_kind=kind,
                            subject_id=subject, dtype=dtype, layout=layout, shape_name=shape.name,
                            dimensions=shape.dimensions(), status="skipped", reason=reason))
    return cases


def run_decode_linear_w4a16_suite(suite: BenchmarkSuite) -> tuple[list[BenchmarkCase], list[str]]:
    from fast_kernels.benchmarking import case_id
    from fast_kernels.ops import (
        arc_w4a16_forward,
        cublaslt_fp16_after_dequant,
        cuda_decode_available,
        dequant_w4a16_to_fp16,
        group_size_for_layout,
        pack_arc_w4a16_packets,
    )

    try:
        import torch
    except ImportError:
        return _skipped(suite, "PyTorch is not installed"), ["Skipped: PyTorch is not installed."]
    if not cuda_decode_available():
        return _skipped(suite, "native module was not built"), ["Skipped: native module unavailable."]
    if not torch.cuda.is_available():
        return _skipped(suite, "no CUDA device"), ["Skipped: no CUDA device (the kernels have no CPU path)."]

    device = torch.device("cuda")
    dtypes = {"fp16": torch.float16, "bf16": torch.bfloat16}
    peak = float(suite.metadata.get("hbm_peak_gbs", DEFAULT_HBM_PEAK_GBS))
    kernels = kernel_registry()
    cases: list[BenchmarkCase] = []

    def emit(kind: str, subject: str, dtype: str, layout: str, shape: ShapeCase, **fields: Any) -> None:
        cases.append(BenchmarkCase(case_id=case_id(kind, subject, dtype, layout, shape.name), subject_kind=kind,
                                   subject_id=subject, dtype=dtype, layout=layout, shape_name=shape.name,
                                   dimensions=shape.dimensions(), **fields))

    subjects = [("baseline", b) for b in suite.baselines.ids] + [("kernel", k) for k in suite.kernels.ids]
    for dtype_name in suite.dtypes:
        for layout in suite.layouts:
            for shape in suite.shapes:
                reason = None
                if dtype_name not in dtypes:
                    reason = f"dtype {dtype_name} is not supported (fp16, bf16)"
                else:
                    try:
                        group = group_size_for_layout(layout)
                    except ValueError as exc:
                        reason = str(exc)
                if reason is None:
                    n, k = shape.n or 0, shape.k or 0
                    if shape.m not in (None, 1):
                        reason = "decode suites carry the GEMV rows in `batch`; m must be 1"
                    elif n <= 0 or n % 128 != 0 or k <= 0 or k % group != 0:
                        reason = "n must be a multiple of 128 and k a multiple of the group size"
                if reason is not None:
                    for kind, subject in subjects:
                        emit(kind, subject, dtype_name, layout, shape, status="skipped", reason=reason)
                    continue

                dtype = dtypes[dtype_name]
                act, q_u8, alpha, beta = _make_inputs(torch, suite, shape, group, dtype, device)
                packets = pack_arc_w4a16_packets(q_u8, alpha, beta, group_size=group)
                expected = _explicit_reference(torch, act, q_u8, alpha, beta, group)
                copies = max(2, min(16, ROTATION_BYTES // max(1, packets.numel())))
                packet_copies = [packets] + [packets.clone() for _ in range(copies - 1)]
                out = torch.empty_like(expected)
                weight = torch.empty((n, k), dtype=dtype, device=device)
                bytes_moved = n * k // 2 + 4 * n * (k // group) + 2 * shape.batch * (k + n)

                def make_calls(kind: str, subject: str) -> list[Callable[[], Any]]:
                    if kind == "kernel":
                        impl = kernels[subject].impl
                        return [
                            (lambda p=p: arc_w4a16_forward(act, p, n=n, k=k, group_size=group, output=out, impl=impl))
                            for p in packet_copies
                        ]
                    if subject.startswith("vendor/"):
                        return [lambda: cublaslt_fp16_after_dequant(act, q_u8, alpha, beta, group_size=group,
                                                                    output=out, weight_buffer=weight)]

                    def torch_reference() -> Any:
                        dequant_w4a16_to_fp16(q_u8, alpha, beta, group_size=group, output=weight)
                        return torch.mm(act, weight.t(), out=out)

                    return [torch_reference]

                timings: dict[str, float] = {}
                pending: list[tuple[str, str, dict[str, Any]]] = []
                for kind, subject in subjects:
                    try:
                        calls = make_calls(kind, subject)
                        out.fill_(float("nan"))
                        calls[-1]()
                        torch.cuda.synchronize()
                        diff = (out.float() - expected.float()).abs()
                        max_err = float(diff.max().item())
                        if not bool(torch.allclose(out, expected, atol=suite.tolerances.atol, rtol=suite.tolerances.rtol)):
                            raise AssertionError(f"mismatch vs explicit fp32 reference: max_abs_diff={max_err:.6f}")
                        device_us = _time_device(torch, calls, TIMING_ITERS)
                        wall_us = _time_wall(torch, calls)
                    except Exception as exc:  # noqa: BLE001 - a failing subject must not stop the suite
                        emit(kind, subject, dtype_name, layout, shape, status="failed", reason=f"{type(exc).__name__}: {exc}")
                        continue
                    dev_med = float(median(device_us))
                    timings[subject] = dev_med
                    gbs = bytes_moved / (dev_med * 1e-6) / 1e9
                    pending.append((kind, subject, {
                        "status": "ok",
                        "latency_us_median": dev_med,
                        "latency_us_p95": _p95(device_us),
                        "device_latency_us_median": dev_med,
                        "device_latency_us_p95": _p95(device_us),
                        "wall_latency_us_median": float(median(wall_us)),
                        "wall_latency_us_p95": _p95(wall_us),
                        "throughput": shape.batch * 1e6 / dev_med,
                        "decode_tokens_per_second": shape.batch * 1e6 / dev_med,
                        "metrics": {"hbm_gbs": gbs, "hbm_frac_of_measured_peak": gbs / peak,
                                    "algorithmic_bytes": float(bytes_moved), "max_abs_err": max_err,
                                    "weight_copies_rotated": float(len(calls))},
                    }))
                for kind, subject, fields in pending:
                    if kind == "kernel":
                        fields["speedup_vs"] = {b: timings[b] / fields["latency_us_median"]
                                                for b in suite.baselines.ids if b in timings}
                    emit(kind, subject, dtype_name, layout, shape, **fields)
                del packet_copies, weight
                torch.cuda.empty_cache()

    notes = [
        "latency_us_* are CUDA-event device times; wall_* include launch overhead and a host sync per call.",
        f"Kernel subjects cycle through up to 16 weight copies (>= {ROTATION_BYTES >> 20} MiB in total where they "
        "fit) so weights come from HBM, not L2; baselines re-read one copy.",
        f"hbm_frac_of_measured_peak uses {peak:.1f} GB/s.",
    ]
    return cases, notes
