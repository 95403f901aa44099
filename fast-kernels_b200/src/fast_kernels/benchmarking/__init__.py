"""``load_suite`` / ``verify_suite`` / ``benchmark_suite``: what ``fk verify`` and ``fk bench`` call.

Same contract as the reference's runner (src/fast_kernels/benchmarking/runner.py:31-151): a suite
is valid when every kernel and baseline id is registered and shapes, dtypes and layouts are
non-empty; a bench run validates first, then writes
``<root>/<suite.id>/<run_id>/{metadata.json,results.json,results.csv,summary.md,plots/status_counts.svg}``.
Suites of the ``decode_quant_linear`` family are executed (the reference dispatches on the one suite
id ``decode_linear_w4a16``; widening to the family lets the added bf16 / edge-shape suites run);
suites of the ``clustered_page_decode`` family likewise; any other suite yields ``not_implemented``
cases, as the reference's scaffold path does.
"""

from __future__ import annotations

import tomllib
from collections import Counter
from datetime import UTC, datetime
from pathlib import Path

from fast_kernels.env import collect_environment
from fast_kernels.registry import baseline_registry, kernel_registry
from fast_kernels.reporting import write_result_bundle
from fast_kernels.schemas import BenchmarkCase, BenchmarkSuite, ResultBundle, RunMetadata

__all__ = ["benchmark_suite", "case_id", "load_suite", "summarize_statuses", "verify_suite"]


def load_suite(path: str | Path) -> BenchmarkSuite:
    with Path(path).open("rb") as handle:
        return BenchmarkSuite.model_validate(tomllib.load(handle))


def verify_suite(suite: BenchmarkSuite) -> list[str]:
    errors: list[str] = []
    if not suite.kernels.ids:
        errors.append("suite defines no kernels")
    if not suite.baselines.ids:
        errors.append("suite defines no baselines")
    known_kernels, known_baselines = kernel_registry(), baseline_registry()
    errors += [f"unknown kernel id: {kid}" for kid in suite.kernels.ids if kid not in known_kernels]
    errors += [f"unknown baseline id: {bid}" for bid in suite.baselines.ids if bid not in known_baselines]
    for field in ("shapes", "dtypes", "layouts"):
        if not getattr(suite, field):
            errors.append(f"suite defines no {field}")
    return errors


def case_id(kind: str, subject_id: str, dtype: str, layout: str, shape_name: str) -> str:
    return f"{kind}-{subject_id.replace('/', '__')}-{dtype}-{layout}-{shape_name}"


def _scaffold_cases(suite: BenchmarkSuite) -> list[BenchmarkCase]:
    cases = []
    for kind, ids in (("kernel", suite.kernels.ids), ("baseline", suite.baselines.ids)):
        for subject in ids:
            for dtype in suite.dtypes:
                for layout in suite.layouts:
                    for shape in suite.shapes:
                        cases.append(BenchmarkCase(
                            case_id=case_id(kind, subject, dtype, layout, shape.name), subject_kind=kind,
                            subject_id=subject, dtype=dtype, layout=layout, shape_name=shape.name,
                            dimensions=shape.dimensions(), status="not_implemented",
                            reason=f"{subject} is registered but has no runner in this build",
                        ))
    return cases


def _execute(suite: BenchmarkSuite) -> tuple[list[BenchmarkCase], list[str]]:
    if suite.family == "decode_quant_linear":
        from fast_kernels.benchmarking.decode_linear_w4a16 import run_decode_linear_w4a16_suite

        return run_decode_linear_w4a16_suite(suite)
    if suite.family in ("clustered_page_decode", "prefix_union_decode"):
        from fast_kernels.benchmarking.clustered_page_decode import run_clustered_page_decode_suite

        return run_clustered_page_decode_suite(suite)
    return _scaffold_cases(suite), ["Scaffold run: this suite's family has no runner in this build."]


def benchmark_suite(suite_path: str | Path, output_root: str | Path | None = None) -> Path:
    suite = load_suite(suite_path)
    errors = verify_suite(suite)
    if errors:
        raise ValueError("Suite validation failed:\n" + "\n".join(f"- {error}" for error in errors))
    env = collect_environment(Path(suite_path).resolve().parent)
    now = datetime.now(tz=UTC)
    run_id = f"{now.strftime('%Y%m%dT%H%M%SZ')}-{env.git_sha or 'worktree'}"
    cases, notes = _execute(suite)
    metadata = RunMetadata(
        run_id=run_id, suite_id=suite.id, created_at=now.isoformat(), git_sha=env.git_sha,
        python_version=env.python_version, platform=env.platform, machine=env.machine, native=env.native,
        nvidia_smi=env.nvidia_smi, nvcc_version=env.nvcc_version, torch_version=env.torch_version, notes=notes,
    )
    root = Path(output_root) if output_root is not None else Path.cwd() / "results"
    run_dir = root / suite.id / run_id
    write_result_bundle(run_dir, ResultBundle(metadata=metadata, cases=cases))
    return run_dir


def summarize_statuses(bundle: ResultBundle) -> dict[str, int]:
    return dict(Counter(case.status for case in bundle.cases))
