"""``fk env | verify | bench | report | plot`` -- the reference's commands and exit codes
(src/fast_kernels/cli/main.py:17-117), printed with plain text instead of rich tables."""

from __future__ import annotations

import argparse
from collections.abc import Sequence
from pathlib import Path

from fast_kernels.benchmarking import benchmark_suite, load_suite, verify_suite
from fast_kernels.env import collect_environment
from fast_kernels.reporting import load_result_bundle, render_plot, render_summary_markdown


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="fk", description="fast-kernels development CLI")
    sub = parser.add_subparsers(dest="command", required=True)
    env = sub.add_parser("env", help="Print environment and build information.")
    env.add_argument("--json", action="store_true", help="Emit JSON instead of a table.")
    verify = sub.add_parser("verify", help="Validate a benchmark suite.")
    verify.add_argument("suite", type=Path)
    bench = sub.add_parser("bench", help="Run a benchmark suite and write result artifacts.")
    bench.add_argument("suite", type=Path)
    bench.add_argument("--output-root", type=Path, default=None)
    report = sub.add_parser("report", help="Regenerate summary markdown for a run.")
    report.add_argument("run_dir", type=Path)
    plot = sub.add_parser("plot", help="Regenerate SVG plots for a run.")
    plot.add_argument("run_dir", type=Path)
    return parser


def main(argv: Sequence[str] | None = None) -> int:
    args = _parser().parse_args(list(argv) if argv is not None else None)
    if args.command == "env":
        snapshot = collect_environment()
        if args.json:
            print(snapshot.to_json())
        else:
            for key, value in vars(snapshot).items():
                print(f"{key:16s} {value}")
        return 0
    if args.command == "verify":
        suite = load_suite(args.suite)
        errors = verify_suite(suite)
        if errors:
            print("Suite validation failed:")
            for error in errors:
                print(f"- {error}")
            return 1
        print(f"Suite valid: {suite.id}")
        print(f"{len(suite.kernels.ids)} kernels, {len(suite.baselines.ids)} baselines, {len(suite.shapes)} shapes.")
        return 0
    if args.command == "bench":
        print(f"Wrote benchmark run to {benchmark_suite(args.suite, args.output_root)}")
        return 0
    bundle = load_result_bundle(args.run_dir)
    if args.command == "report":
        target = Path(args.run_dir) / "summary.md"
        target.write_text(render_summary_markdown(bundle), encoding="utf-8")
    else:
        target = render_plot(bundle, Path(args.run_dir) / "plots" / "status_counts.svg")
    print(f"Updated {target}")
    return 0


if __name__ == "__main__":  # pragma: no cover
    raise SystemExit(main())
