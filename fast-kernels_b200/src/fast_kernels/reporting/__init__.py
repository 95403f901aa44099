"""Result artifacts of a run: metadata.json, results.json, results.csv, summary.md and
plots/status_counts.svg -- the five files the reference's ``fk bench`` leaves
(src/fast_kernels/reporting/artifacts.py:48-77). The SVG is written directly (no plotting library)."""

from __future__ import annotations

import csv
import json
from collections import Counter
from pathlib import Path

from fast_kernels.schemas import BenchmarkCase, ResultBundle, RunMetadata

__all__ = ["load_result_bundle", "render_plot", "render_summary_markdown", "write_result_bundle"]

_CSV_FIELDS = [
    "case_id", "subject_kind", "subject_id", "dtype", "layout", "shape_name", "status",
    "latency_us_median", "latency_us_p95", "device_latency_us_median", "wall_latency_us_median",
    "decode_tokens_per_second", "hbm_gbs", "hbm_frac_of_measured_peak", "max_abs_err", "reason",
]


def _fmt(value: float | None, digits: int = 2) -> str:
    return "-" if value is None else f"{value:.{digits}f}"


def render_summary_markdown(bundle: ResultBundle) -> str:
    meta = bundle.metadata
    counts = Counter(case.status for case in bundle.cases)
    lines = [
        f"# {meta.suite_id} - run {meta.run_id}",
        "",
        f"- created: {meta.created_at}",
        f"- git: {meta.git_sha or 'worktree'}; torch {meta.torch_version or '-'}; nvcc {meta.nvcc_version or '-'}",
        f"- gpu: {(meta.nvidia_smi or {}).get('name', 'none')}",
        "- statuses: " + ", ".join(f"{name}={count}" for name, count in sorted(counts.items())),
        "",
    ]
    lines += [f"> {note}" for note in meta.notes]
    lines += [
        "",
        "| subject | dtype | layout | shape | status | device us | wall us | tok/s | GB/s | of peak | speed-up vs vendor |",
        "|---|---|---|---|---|---|---|---|---|---|---|",
    ]
    for case in bundle.cases:
        vendor = next((v for key, v in case.speedup_vs.items() if key.startswith("vendor/")), None)
        lines.append(
            f"| {case.subject_id} | {case.dtype} | {case.layout} | {case.shape_name} | {case.status} | "
            f"{_fmt(case.device_latency_us_median)} | {_fmt(case.wall_latency_us_median)} | "
            f"{_fmt(case.decode_tokens_per_second, 0)} | {_fmt(case.metrics.get('hbm_gbs'), 0)} | "
            f"{_fmt(case.metrics.get('hbm_frac_of_measured_peak'), 3)} | {_fmt(vendor)} |"
        )
    return "\n".join(lines) + "\n"


def render_plot(bundle: ResultBundle, destination: str | Path) -> Path:
    """Bar chart of case statuses as a small hand-written SVG."""
    path = Path(destination)
    path.parent.mkdir(parents=True, exist_ok=True)
    counts = Counter(case.status for case in bundle.cases)
    colours = {"ok": "#2e7d32", "skipped": "#9e9e9e", "not_implemented": "#f9a825", "failed": "#c62828"}
    peak = max(counts.values(), default=1)
    bars = []
    for index, (status, count) in enumerate(sorted(counts.items())):
        height = 160 * count / peak
        x = 40 + index * 110
        bars.append(
            f'<rect x="{x}" y="{200 - height:.1f}" width="80" height="{height:.1f}" '
            f'fill="{colours.get(status, "#455a64")}"/>'
            f'<text x="{x + 40}" y="216" font-size="11" text-anchor="middle">{status}</text>'
            f'<text x="{x + 40}" y="{194 - height:.1f}" font-size="11" text-anchor="middle">{count}</text>'
        )
    width = 80 + 110 * max(len(counts), 1)
    svg = (
        f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="230" font-family="sans-serif">'
        f'<text x="10" y="18" font-size="13">{bundle.metadata.suite_id}: case statuses</text>'
        + "".join(bars) + "</svg>\n"
    )
    path.write_text(svg, encoding="utf-8")
    return path


def write_result_bundle(run_dir: str | Path, bundle: ResultBundle) -> Path:
    root = Path(run_dir)
    root.mkdir(parents=True, exist_ok=True)
    (root / "metadata.json").write_text(bundle.metadata.model_dump_json(indent=2) + "\n", encoding="utf-8")
    (root / "results.json").write_text(bundle.model_dump_json(indent=2) + "\n", encoding="utf-8")
    with (root / "results.csv").open("w", newline="", encoding="utf-8") as handle:
        writer = csv.DictWriter(handle, fieldnames=_CSV_FIELDS)
        writer.writeheader()
        for case in bundle.cases:
            row = {key: getattr(case, key, None) for key in _CSV_FIELDS if hasattr(case, key)}
            for key in ("hbm_gbs", "hbm_frac_of_measured_peak", "max_abs_err"):
                row[key] = case.metrics.get(key)
            writer.writerow(row)
    (root / "summary.md").write_text(render_summary_markdown(bundle), encoding="utf-8")
    render_plot(bundle, root / "plots" / "status_counts.svg")
    return root


def load_result_bundle(run_dir: str | Path) -> ResultBundle:
    root = Path(run_dir)
    payload = json.loads((root / "results.json").read_text(encoding="utf-8"))
    bundle = ResultBundle.model_validate(payload)
    assert isinstance(bundle.metadata, RunMetadata) and all(isinstance(c, BenchmarkCase) for c in bundle.cases)
    return bundle
