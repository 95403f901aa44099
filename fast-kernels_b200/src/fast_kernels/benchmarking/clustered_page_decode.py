"""Runner for suites of the ``clustered_page_decode`` and ``prefix_union_decode`` families (what
``fk bench`` executes for them).

Same flow as the reference's runner for this family
(src/fast_kernels/benchmarking/clustered_page_decode.py there): per layout x shape it draws seeded
queries, keys and values (sequence lengths within one page of ``max_seq_len``), pages them behind a
fragmented page table, plans, gates every subject on agreement with the PyTorch reference under
the suite's tolerances and then times it. ``decode/clustered_page_decode_{auto,direct,clustered}``
are the op with ``force_impl`` = auto / direct / clustered; ``torch/reference_clustered_page_decode``
is the PyTorch statement of the op; ``vendor/flashinfer_clustered_page_decode`` is reported as
skipped (that library's paged decode takes another cache layout and applies no rotary embedding,
and nothing here converts for it). Latencies are CUDA-event device times over CUDA-graph replays
that cycle through enough copies of the pages to exceed L2. Without a GPU every case is skipped.

``prefix_union_decode`` suites (the reference's runner: src/fast_kernels/benchmarking/prefix_union_decode.py
there) use the same flow with the shared-prefix recipe: groups of ``prefix_group_size`` requests
repeat their leader's first ``shared_prefix_pages`` pages, identical pages are stored once, keys
are rotated ahead of time. ``decode/prefix_union_decode_{auto,fallback}`` are the op with that
``force_impl``; ``decode/prefix_union_decode_union`` is skipped with the reference's own reason (its
union kernel needs compute capability 12).
"""

from __future__ import annotations

import importlib
from statistics import median
from typing import Any

from fast_kernels.schemas import BenchmarkCase, BenchmarkSuite, ShapeCase

TIMING_ITERS = 12
ROTATION_BYTES = 512 * 1024 * 1024
DEFAULT_HBM_PEAK_GBS = 6542.7
FORCE_IMPL = {
    "decode/clustered_page_decode_auto": "auto",
    "decode/clustered_page_decode_direct": "direct",
    "decode/clustered_page_decode_clustered": "clustered",
    "decode/prefix_union_decode_auto": "auto",
    "decode/prefix_union_decode_union": "union",
    "decode/prefix_union_decode_fallback": "fallback",
}


def _cases(suite: BenchmarkSuite, status: str, reason: str) -> list[BenchmarkCase]:
    from fast_kernels.benchmarking import case_id

    return [
        BenchmarkCase(case_id=case_id(kind, subject, dtype, layout, shape.name), subject_kind=kind, subject_id=subject,
                      dtype=dtype, layout=layout, shape_name=shape.name, dimensions=shape.dimensions(), status=status,
                      reason=reason)
        for kind, ids in (("kernel", suite.kernels.ids), ("baseline", suite.baselines.ids))
        for subject in ids for dtype in suite.dtypes for layout in suite.layouts for shape in suite.shapes
    ]


def _p95(samples: list[float]) -> float:
    ordered = sorted(samples)
    return ordered[min(len(ordered) - 1, int(round(0.95 * (len(ordered) - 1))))]


def run_clustered_page_decode_suite(suite: BenchmarkSuite) -> tuple[list[BenchmarkCase], list[str]]:
    from fast_kernels.benchmarking import case_id
    from fast_kernels.benchmarking.decode_linear_w4a16 import _time_device

    ops = importlib.import_module("fast_kernels.ops.clustered_page_decode")
    union = importlib.import_module("fast_kernels.ops.prefix_union_decode")
    shared_prefixes = suite.family == "prefix_union_decode"
    try:
        import torch
    except ImportError:
        return _cases(suite, "skipped", "PyTorch is not installed"), ["Skipped: PyTorch is not installed."]
    if not ops.cuda_clustered_decode_available():
        return _cases(suite, "skipped", "native module was not built"), ["Skipped: native module unavailable."]
    if not torch.cuda.is_available():
        return _cases(suite, "skipped", "no CUDA device"), ["Skipped: no CUDA device (the kernel has no CPU path)."]

    device = torch.device("cuda")
    peak = float(suite.metadata.get("hbm_peak_gbs", DEFAULT_HBM_PEAK_GBS))
    builders = {"bf16_kv": ops.pack_paged_kv_bf16, "fp8_kv": ops.quantize_paged_kv_fp8,
                "int8_kv": ops.quantize_paged_kv_int8}
    cases: list[BenchmarkCase] = []

    def emit(kind: str, subject: str, dtype: str, layout: str, shape: ShapeCase, **fields: Any) -> None:
        cases.append(BenchmarkCase(case_id=case_id(kind, subject, dtype, layout, shape.name), subject_kind=kind,
                                   subject_id=subject, dtype=dtype, layout=layout, shape_name=shape.name,
                                   dimensions=shape.dimensions(), **fields))

    subjects = [("baseline", b) for b in suite.baselines.ids] + [("kernel", k) for k in suite.kernels.ids]
    for dtype_name in suite.dtypes:
        for layout in suite.layouts:
            for shape in suite.shapes:
                extra = shape.model_extra or {}
                try:
                    if dtype_name != "bf16":
                        raise ValueError("queries and outputs are bf16")
                    if layout not in builders:
                        raise ValueError(f"layout must be one of {sorted(builders)}")
                    page, max_len = int(extra["page_size"]), int(extra["max_seq_len"])
                    q_heads, kv_heads, dim = int(extra["num_q_heads"]), int(extra["num_kv_heads"]), int(extra["head_dim"])
                except (KeyError, ValueError) as exc:
                    for kind, subject in subjects:
                        emit(kind, subject, dtype_name, layout, shape, status="skipped", reason=f"{exc}")
                    continue
                batch = int(shape.batch)
                shared_pages, group = int(extra.get("shared_prefix_pages", 0)), int(extra.get("prefix_group_size", 1))
                torch.manual_seed(batch + q_heads + kv_heads + dim + max_len + page + shared_pages + group * shared_prefixes)
                query = torch.randn((batch, q_heads, dim), device=device).to(torch.bfloat16)
                keys = torch.randn((batch, kv_heads, max_len, dim), device=device).to(torch.bfloat16)
                values = torch.randn((batch, kv_heads, max_len, dim), device=device).to(torch.bfloat16)
                if shared_prefixes:
                    shared_tokens = shared_pages * page
                    lens = torch.randint(max(page, shared_tokens + 1), max_len + 1, (batch,), dtype=torch.int32)
                    for start in range(0, batch, max(1, group)):
                        keys[start + 1 : start + group, :, :shared_tokens] = keys[start, :, :shared_tokens]
                        values[start + 1 : start + group, :, :shared_tokens] = values[start, :, :shared_tokens]
                    cache = builders[layout](keys, values, lens, page_size=page, fragment_pages=True, seed=3,
                                             key_rope_theta=10000.0, deduplicate_identical_pages=True)
                    union_plan = union.plan_prefix_union_decode(
                        page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=q_heads,
                        num_kv_heads=kv_heads, head_dim=dim, page_size=page, kv_layout=layout, keys_are_rotated=True)
                    plan = union_plan.fallback_plan
                else:
                    lens = torch.randint(max(page, max_len - page + 1), max_len + 1, (batch,), dtype=torch.int32)
                    cache = builders[layout](keys, values, lens, page_size=page, fragment_pages=True, seed=1)
                    plan = ops.plan_clustered_page_decode(page_table=cache.page_table, seq_lens=cache.seq_lens,
                                                          num_q_heads=q_heads, num_kv_heads=kv_heads, head_dim=dim,
                                                          page_size=page, kv_layout=layout)
                expected = ops.reference_clustered_page_decode(query, cache)
                tokens = int(lens.sum())
                element = 2 if layout == "bf16_kv" else 1
                bytes_moved = tokens * kv_heads * dim * 2 * element + 4 * query.numel()
                if element == 1:
                    bytes_moved += (tokens + cache.total_pages) * kv_heads * (dim // 64) * 4
                page_bytes = 2 * cache.key_pages.numel() * cache.key_pages.element_size()
                copies = max(2, min(32, ROTATION_BYTES // max(1, page_bytes)))
                caches = [cache] + [
                    ops.PagedKVCache(
                        key_pages=cache.key_pages.clone(), value_pages=cache.value_pages.clone(),
                        page_table=cache.page_table, seq_lens=cache.seq_lens, key_scales=cache.key_scales,
                        value_scales=cache.value_scales, reference_key_pages=cache.reference_key_pages,
                        reference_value_pages=cache.reference_value_pages, kv_layout=cache.kv_layout,
                        page_size=cache.page_size, num_kv_heads=cache.num_kv_heads, head_dim=cache.head_dim,
                        keys_are_rotated=cache.keys_are_rotated, key_rope_theta=cache.key_rope_theta)
                    for _ in range(copies - 1)
                ]
                out = torch.empty_like(query)
                timings: dict[str, float] = {}
                pending: list[tuple[str, str, dict[str, Any]]] = []
                for kind, subject in subjects:
                    if subject.startswith("vendor/"):
                        emit(kind, subject, dtype_name, layout, shape, status="skipped",
                             reason="no converter to that library's cache layout in this build")
                        continue
                    try:
                        if kind == "kernel":
                            impl = FORCE_IMPL[subject]
                            if impl == "direct" and q_heads // kv_heads > 8:
                                emit(kind, subject, dtype_name, layout, shape, status="skipped",
                                     reason='force_impl="direct" only supports group_size <= 8')
                                continue
                            if impl == "union":
                                emit(kind, subject, dtype_name, layout, shape, status="skipped",
                                     reason="prefix_union_decode requires a Blackwell-class GPU for union mode "
                                            "(compute capability 12, the reference's rule)")
                                continue
                            if shared_prefixes:
                                calls = [(lambda c=c: union.prefix_union_decode(query, c, plan=union_plan, output=out,
                                                                                force_impl=impl)) for c in caches]
                            else:
                                calls = [(lambda c=c: ops.clustered_page_decode(query, c, plan=plan, output=out,
                                                                                force_impl=impl)) for c in caches]
                        else:
                            calls = [lambda: ops.reference_clustered_page_decode(query, cache, output=out)]
                        out.fill_(float("nan"))
                        calls[-1]()
                        torch.cuda.synchronize()
                        max_err = float((out.float() - expected.float()).abs().max().item())
                        if not bool(torch.allclose(out, expected, atol=suite.tolerances.atol, rtol=suite.tolerances.rtol)):
                            raise AssertionError(f"mismatch vs the PyTorch reference: max_abs_diff={max_err:.6f}")
                        iters = TIMING_ITERS if kind == "kernel" else 2
                        device_us = _time_device(torch, calls, iters)
                    except Exception as exc:  # noqa: BLE001 - a failing subject must not stop the suite
                        emit(kind, subject, dtype_name, layout, shape, status="failed", reason=f"{type(exc).__name__}: {exc}")
                        continue
                    dev_med = float(median(device_us))
                    timings[subject] = dev_med
                    gbs = bytes_moved / (dev_med * 1e-6) / 1e9
                    pending.append((kind, subject, {
                        "status": "ok", "latency_us_median": dev_med, "latency_us_p95": _p95(device_us),
                        "device_latency_us_median": dev_med, "device_latency_us_p95": _p95(device_us),
                        "throughput": batch * 1e6 / dev_med, "decode_tokens_per_second": batch * 1e6 / dev_med,
                        "metrics": {"hbm_gbs": gbs, "hbm_frac_of_measured_peak": gbs / peak,
                                    "algorithmic_bytes": float(bytes_moved), "max_abs_err": max_err,
                                    "context_tokens": float(tokens),
                                    **(union.estimate_prefix_union_decode_metrics(cache, union_plan) if shared_prefixes
                                       else ops.estimate_page_decode_metrics(cache, plan))},
                    }))
                for kind, subject, fields in pending:
                    if kind == "kernel":
                        fields["speedup_vs"] = {b: timings[b] / fields["latency_us_median"]
                                                for b in suite.baselines.ids if b in timings}
                    emit(kind, subject, dtype_name, layout, shape, **fields)
                del caches, keys, values
                torch.cuda.empty_cache()
    notes = [
        "latency_us_* are CUDA-event device times over CUDA-graph replays.",
        f"Kernel subjects cycle through copies of the pages (up to {ROTATION_BYTES >> 20} MiB in total) so that "
        "keys and values come from HBM; the PyTorch baseline is eager and re-reads one copy.",
        f"hbm_frac_of_measured_peak uses {peak:.1f} GB/s; decode_tokens_per_second counts one new token per request.",
    ]
    return cases, notes
