"""The suite / CLI contract (`fk verify`, `fk bench`), checked on CPU the way the reference's own
tests do (tests/python/test_suites.py:18-34, test_decode_benchmark.py:13-23, test_cli.py:11-30,
tests/reporting/test_artifacts.py:10-42 in SamMausberg/fast-kernels)."""

from __future__ import annotations

import json
from pathlib import Path

import pytest
from fast_kernels.benchmarking import benchmark_suite, load_suite, verify_suite
from fast_kernels.cli.main import main as fk_main
from fast_kernels.reporting import load_result_bundle, write_result_bundle
from fast_kernels.schemas import BenchmarkCase, ResultBundle, RunMetadata

SUITES = Path(__file__).resolve().parent.parent / "fast-kernels_b200" / "benchmarks" / "suites"


def test_stock_decode_suite_keeps_the_reference_contract() -> None:
    suite = load_suite(SUITES / "decode_linear_w4a16.toml")
    assert suite.id == "decode_linear_w4a16" and suite.family == "decode_quant_linear"
    assert suite.kernels.ids == ["decode/w4a16_linear", "decode/w4a16_linear_scalar",
                                 "decode/w4a16_linear_tc", "decode/w4a16_linear_wgmma"]
    assert "vendor/cublaslt_fp16_after_dequant" in suite.baselines.ids
    assert "groupwise_64" in suite.layouts
    assert len(suite.shapes) == 12
    assert suite.tolerances.atol == 0.0625 and suite.tolerances.rtol == 0.01
    assert verify_suite(suite) == []


@pytest.mark.parametrize("name", sorted(p.name for p in SUITES.glob("*.toml")))
def test_every_shipped_suite_verifies(name: str) -> None:
    assert verify_suite(load_suite(SUITES / name)) == []


def test_verify_reports_unknown_ids_and_empty_sections(tmp_path: Path) -> None:
    bad = tmp_path / "bad.toml"
    bad.write_text('id = "x"\nfamily = "decode_quant_linear"\ndescription = "d"\n'
                   '[kernels]\nids = ["decode/nope"]\n[baselines]\nids = []\n')
    errors = verify_suite(load_suite(bad))
    assert "unknown kernel id: decode/nope" in errors
    assert "suite defines no baselines" in errors and "suite defines no shapes" in errors
    assert fk_main(["verify", str(bad)]) == 1
    with pytest.raises(ValueError, match="Suite validation failed"):
        benchmark_suite(bad, tmp_path)


def test_decode_bench_writes_a_bundle_without_a_gpu(tmp_path: Path) -> None:
    run_dir = benchmark_suite(SUITES / "decode_linear_w4a16.toml", tmp_path)
    bundle = load_result_bundle(run_dir)
    assert bundle.schema_version == 2 and bundle.metadata.suite_id == "decode_linear_w4a16"
    assert len(bundle.cases) == (4 + 2) * 1 * 2 * 12
    assert {case.status for case in bundle.cases} <= {"ok", "skipped", "failed"}
    assert (run_dir / "summary.md").exists()
    first = bundle.cases[0]
    assert first.case_id == "kernel-decode__w4a16_linear-fp16-groupwise_64-llama_qkv_bs1"


def test_page_decode_suite_keeps_the_reference_contract_and_benches(tmp_path: Path) -> None:
    """Ids, shapes and tolerances of the reference's benchmarks/suites/clustered_page_decode.toml; the
    bench writes one case per subject x layout x shape (skipped without a GPU, never silently run on
    the CPU)."""
    suite = load_suite(SUITES / "clustered_page_decode.toml")
    assert suite.id == "clustered_page_decode" and suite.family == "clustered_page_decode"
    assert suite.kernels.ids == ["decode/clustered_page_decode_auto", "decode/clustered_page_decode_direct",
                                 "decode/clustered_page_decode_clustered"]
    assert suite.baselines.ids == ["torch/reference_clustered_page_decode", "vendor/flashinfer_clustered_page_decode"]
    assert suite.layouts == ["bf16_kv", "fp8_kv", "int8_kv"] and [s.name for s in suite.shapes] == [
        "gqa4_short_page16", "gqa4_long_page16", "mqa8_long_page32", "mqa32_long_page32", "gqa2_short_page32_h64"]
    assert suite.shapes[3].dimensions()["num_kv_heads"] == 1 and suite.shapes[3].dimensions()["max_seq_len"] == 4096
    assert suite.tolerances.atol == 0.125 and suite.tolerances.rtol == 0.03
    run_dir = benchmark_suite(SUITES / "clustered_page_decode.toml", tmp_path)
    bundle = load_result_bundle(run_dir)
    assert len(bundle.cases) == (3 + 2) * 1 * 3 * 5
    assert {case.status for case in bundle.cases} <= {"ok", "skipped", "failed"}


def test_prefix_union_suite_keeps_the_reference_contract(tmp_path: Path) -> None:
    suite = load_suite(SUITES / "prefix_union_decode.toml")
    assert suite.family == "prefix_union_decode" and suite.kernels.ids == [
        "decode/prefix_union_decode_auto", "decode/prefix_union_decode_union", "decode/prefix_union_decode_fallback"]
    assert suite.baselines.ids == ["torch/reference_prefix_union_decode"]
    assert [s.name for s in suite.shapes] == ["gqa4_prefix4_page16", "gqa4_prefix8_page16", "mqa8_prefix8_page32",
                                              "gqa2_prefix4_page32_h64"]
    assert suite.shapes[1].dimensions()["shared_prefix_pages"] == 8
    bundle = load_result_bundle(benchmark_suite(SUITES / "prefix_union_decode.toml", tmp_path))
    assert len(bundle.cases) == (3 + 1) * 1 * 3 * 4 and {case.status for case in bundle.cases} <= {"ok", "skipped", "failed"}


def test_cli_env_and_template_bench(tmp_path: Path, capsys: pytest.CaptureFixture[str]) -> None:
    assert fk_main(["env", "--json"]) == 0
    payload = json.loads(capsys.readouterr().out)
    assert "python_version" in payload and "native" in payload
    assert fk_main(["bench", str(SUITES / "template_gemm.toml"), "--output-root", str(tmp_path)]) == 0
    run_dir = next((tmp_path / "template_gemm").iterdir())
    for artifact in ("metadata.json", "results.json", "results.csv", "summary.md", "plots/status_counts.svg"):
        assert (run_dir / artifact).exists(), artifact
    assert {c.status for c in load_result_bundle(run_dir).cases} == {"not_implemented"}
    assert fk_main(["report", str(run_dir)]) == 0 and fk_main(["plot", str(run_dir)]) == 0
    assert fk_main(["verify", str(SUITES / "w4a16_llama3_8b_m1.toml")]) == 0


def test_result_bundle_round_trip(tmp_path: Path) -> None:
    meta = RunMetadata(run_id="r1", suite_id="s", created_at="now", python_version="3", platform="p", machine="m")
    case = BenchmarkCase(case_id="c", subject_kind="kernel", subject_id="decode/w4a16_linear", dtype="bf16",
                         layout="groupwise_128", shape_name="qkv", dimensions={"n": 6144, "k": 4096, "batch": 1},
                         status="ok", latency_us_median=6.3, metrics={"hbm_gbs": 2100.0})
    write_result_bundle(tmp_path, ResultBundle(metadata=meta, cases=[case]))
    loaded = load_result_bundle(tmp_path)
    assert loaded.schema_version == 2 and loaded.cases[0].metrics["hbm_gbs"] == 2100.0
    assert "decode/w4a16_linear" in (tmp_path / "summary.md").read_text()
