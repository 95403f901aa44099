"""Paged-KV decode attention, the parts that need no GPU: the fp64 oracle against the fixtures the
reference's own Python produced, this package's host-side preparation (paging, quantisation,
planning, PyTorch reference) against the same fixtures, and the C-ABI surface."""

from __future__ import annotations

import ctypes
import importlib
import re
from pathlib import Path

import numpy as np
import pytest
import torch
from fast_kernels import page_decode_capi as pdc
from oracle import page_decode_oracle as oracle
from page_decode_testlib import KV_IDS, load_case, manifest, oracle_on_case

REPO = Path(__file__).resolve().parent.parent
ops = importlib.import_module("fast_kernels.ops.clustered_page_decode")
CASES = manifest()
IDS = [m["name"] for m in CASES]


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


# ---- the oracle is pinned by the reference's PyTorch reference ------------------------------------
@pytest.mark.parametrize("meta", CASES, ids=IDS)
def test_oracle_agrees_with_the_reference_outputs(meta) -> None:
    case = load_case(meta["name"])
    got = oracle_on_case(oracle, meta, case)
    expected = oracle.bf16_bits_to_f64(case["expected"])
    if meta["layout"] == "bf16_kv":
        # same data, fp64 against fp32 + one bf16 rounding of the result (2^-9 relative); keys that
        # were rotated ahead of time carry their own bf16 rounding in both
        _, scaled = oracle.max_abs_and_scaled_error(got, expected, atol=1e-3, rtol=4e-3)
    else:
        # the reference's expectation is computed from the UNQUANTISED pages: its own tolerance
        # (tests/gpu/test_clustered_page_decode.py:156 there) is what separates the two
        _, scaled = oracle.max_abs_and_scaled_error(got, expected, atol=1.25e-1, rtol=3e-2)
    assert scaled <= 1.0


@pytest.mark.parametrize("meta", [m for m in CASES if m["layout"] != "bf16_kv"], ids=lambda m: m["name"])
def test_oracle_on_the_unquantised_pages_is_tight(meta) -> None:
    """The quantised fixtures also hold the bf16 pages the expectation was computed from: on those
    the oracle must agree to rounding, which pins the walk over runs, positions and rotation."""
    case = load_case(meta["name"])
    plain = dict(case, key_pages=case["reference_key_pages"], value_pages=case["reference_value_pages"])
    plain.pop("key_scales"), plain.pop("value_scales")
    got = oracle_on_case(oracle, dict(meta, layout="bf16_kv"), plain)
    _, scaled = oracle.max_abs_and_scaled_error(got, oracle.bf16_bits_to_f64(case["expected"]), atol=1e-3, rtol=4e-3)
    assert scaled <= 1.0


def test_oracle_number_formats() -> None:
    assert oracle.E4M3[0x7E] == 448.0 and oracle.E4M3[0x01] == 2.0**-9 and oracle.E4M3[0xB8] == -1.0
    fp8 = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy().astype(np.float64)
    assert np.array_equal(np.nan_to_num(fp8, nan=7.0), np.nan_to_num(oracle.E4M3, nan=7.0))
    x = torch.randn(1000)
    assert np.array_equal(oracle.f32_to_bf16_bits(x.numpy()), _bits(x.to(torch.bfloat16)))


def test_oracle_handles_empty_requests_and_partial_pages() -> None:
    rng = np.random.default_rng(0)
    query = oracle.f32_to_bf16_bits(rng.standard_normal((3, 2, 64)).astype(np.float32))
    pages = oracle.f32_to_bf16_bits(rng.standard_normal((4, 1, 16, 64)).astype(np.float32))
    out = oracle.page_decode_f64(
        query, pages, pages, None, None, np.array([2, 0]), np.array([1, 2]), np.array([0, 0]), np.array([1, 5]),
        np.array([0, 1, 1, 2]), np.array([1, 0, 21]), kv_format=0, keys_are_rotated=True, softmax_scale=0.125,
        rope_theta=10000.0)
    values = oracle.bf16_bits_to_f64(pages)
    assert np.allclose(out[0, 0], values[2, 0, 0])  # one token: the output is that token's value
    assert not out[1].any()                          # no runs: zeros
    assert out[2].any()


# ---- this package's host side produces the reference's bytes ---------------------------------------
def _build(meta, case):
    keys, values = _bf16(case["keys"]), _bf16(case["values"])
    seq_lens = torch.from_numpy(case["seq_lens"].copy())
    build = {"bf16_kv": ops.pack_paged_kv_bf16, "int8_kv": ops.quantize_paged_kv_int8,
             "fp8_kv": ops.quantize_paged_kv_fp8}[meta["layout"]]
    return build(keys, values, seq_lens, page_size=meta["page_size"], fragment_pages=meta["fragment_pages"],
                 seed=meta["seed"], key_rope_theta=meta["key_rope_theta"],
                 deduplicate_identical_pages=meta["deduplicate_identical_pages"])


@pytest.mark.parametrize("meta", CASES, ids=IDS)
def test_paging_quantisation_and_plan_match_the_reference_bit_for_bit(meta) -> None:
    case = load_case(meta["name"])
    cache = _build(meta, case)
    assert cache.kv_layout == meta["layout"] and cache.total_pages == meta["total_pages"]
    assert np.array_equal(cache.page_table.numpy(), case["page_table"])
    if meta["layout"] == "bf16_kv":
        assert np.array_equal(_bits(cache.key_pages), case["key_pages"])
        assert np.array_equal(_bits(cache.value_pages), case["value_pages"])
    else:
        assert np.array_equal(cache.key_pages.view(torch.uint8).numpy(), case["key_pages"])
        assert np.array_equal(cache.value_pages.view(torch.uint8).numpy(), case["value_pages"])
        assert np.array_equal(cache.key_scales.numpy(), case["key_scales"])
        assert np.array_equal(cache.value_scales.numpy(), case["value_scales"])
        assert np.array_equal(_bits(cache.reference_key_pages), case["reference_key_pages"])
    plan = ops.plan_clustered_page_decode(
        page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=meta["num_q_heads"],
        num_kv_heads=meta["num_kv_heads"], head_dim=meta["head_dim"], page_size=meta["page_size"],
        kv_layout=meta["layout"], use_cache=False)
    for name in ("run_base_pages", "run_page_counts", "run_logical_starts", "run_last_page_lens", "request_run_offsets"):
        assert np.array_equal(getattr(plan, f"{name}_cpu").numpy(), case[name]), name
    for key, value in meta["plan"].items():
        assert getattr(plan, key) == value, key


@pytest.mark.parametrize("meta", CASES, ids=IDS)
def test_pytorch_reference_matches_the_reference_outputs(meta) -> None:
    case = load_case(meta["name"])
    cache = _build(meta, case)
    got = ops.reference_clustered_page_decode(_bf16(case["query"]), cache)
    expected = _bf16(case["expected"])
    # batched contractions instead of one matmul per head: the last fp32 bit may differ, i.e. at
    # most one bf16 step on an output
    torch.testing.assert_close(got.float(), expected.float(), atol=2e-3, rtol=8e-3)


def test_plan_heuristics_and_errors(monkeypatch: pytest.MonkeyPatch) -> None:
    """The reference's plan tests (tests/gpu/test_clustered_page_decode.py:284-343 there)."""
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda _device=None: (12, 0))
    plan = ops.plan_clustered_page_decode(
        page_table=torch.arange(128, dtype=torch.int32).view(1, 128), seq_lens=torch.tensor([2048], dtype=torch.int32),
        num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=16, kv_layout="bf16_kv")
    assert (plan.cluster_size, plan.group_tile, plan.q_head_tiles, plan.launch_mode) == (4, 4, 1, "clustered")
    assert plan.num_runs == 1 and plan.run_page_counts_cpu.tolist() == [128]
    plan = ops.plan_clustered_page_decode(
        page_table=torch.arange(128, dtype=torch.int32).view(1, 128), seq_lens=torch.tensor([4096], dtype=torch.int32),
        num_q_heads=32, num_kv_heads=1, head_dim=128, page_size=32, kv_layout="bf16_kv")
    assert (plan.cluster_size, plan.group_tile, plan.q_head_tiles, plan.launch_mode) == (2, 8, 4, "clustered")
    plan = ops.plan_clustered_page_decode(
        page_table=torch.arange(4, dtype=torch.int32).view(1, 4), seq_lens=torch.tensor([64], dtype=torch.int32),
        num_q_heads=16, num_kv_heads=4, head_dim=64, page_size=16, kv_layout="bf16_kv")
    assert (plan.cluster_size, plan.group_tile, plan.q_head_tiles, plan.launch_mode) == (1, 4, 1, "direct")
    with pytest.raises(ValueError, match="head_dim must be 64 or 128"):
        ops.plan_clustered_page_decode(page_table=torch.zeros((1, 1), dtype=torch.int32),
                                       seq_lens=torch.tensor([1]), num_q_heads=4, num_kv_heads=4, head_dim=96,
                                       page_size=16, kv_layout="bf16_kv")
    with pytest.raises(ValueError, match="layout must be one of"):
        ops.plan_clustered_page_decode(page_table=torch.zeros((1, 1), dtype=torch.int32),
                                       seq_lens=torch.tensor([1]), num_q_heads=4, num_kv_heads=4, head_dim=64,
                                       page_size=16, kv_layout="fp4_kv")
    with pytest.raises(ValueError, match="page_size must be 16 or 32"):
        ops.pack_paged_kv_bf16(torch.zeros(1, 1, 8, 64), torch.zeros(1, 1, 8, 64), torch.tensor([8]), page_size=8)


def test_plan_with_an_empty_request_and_metrics() -> None:
    table = torch.tensor([[5, 6, 9], [-1, -1, -1], [2, -1, -1]], dtype=torch.int32)
    plan = ops.plan_clustered_page_decode(page_table=table, seq_lens=torch.tensor([40, 0, 16], dtype=torch.int32),
                                          num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=16,
                                          kv_layout="int8_kv", use_cache=False)
    assert plan.run_base_pages_cpu.tolist() == [5, 9, 2]
    assert plan.run_page_counts_cpu.tolist() == [2, 1, 1]
    assert plan.run_logical_starts_cpu.tolist() == [0, 2, 0]
    assert plan.run_last_page_lens_cpu.tolist() == [16, 8, 16]
    assert plan.request_run_offsets_cpu.tolist() == [0, 2, 2, 3]
    keys = torch.randn(3, 2, 48, 64)
    cache = ops.quantize_paged_kv_int8(keys, keys, torch.tensor([40, 5, 16], dtype=torch.int32), page_size=16, seed=3)
    metrics = ops.estimate_page_decode_metrics(cache, plan)
    assert metrics["hbm_bytes_per_token"] > 0 and metrics["workspace_bytes_per_token"] == 0.0


# ---- C ABI surface -----------------------------------------------------------------------------------
def test_library_exports_what_the_header_declares() -> None:
    header = (REPO / "include" / "fk_page_decode.h").read_text()
    declared = sorted(set(re.findall(r"\b(fk_page_decode_\w+)\s*\(", header)))
    assert declared == sorted(pdc.SIGNATURES)
    lib = ctypes.CDLL(str(pdc.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), name
    fields = re.search(r"typedef struct fk_page_decode_args \{(.*?)\} fk_page_decode_args;", header, re.S).group(1)
    names = re.findall(r"(\w+);", re.sub(r"/\*.*?\*/", "", fields, flags=re.S))
    assert names == [name for name, _ in pdc.PageDecodeArgs._fields_]


def test_argument_errors_come_before_any_launch() -> None:
    """The rules of the reference's launcher (clustered_page_decode.cu:1095-1131 there)."""
    lib = pdc.load_library()

    def call(**changes):
        a = pdc.PageDecodeArgs()
        for name in ("query", "key_pages", "value_pages", "run_base_pages", "run_page_counts", "run_logical_starts",
                     "run_last_page_lens", "request_run_offsets", "seq_lens", "output"):
            setattr(a, name, 4096)
        a.batch, a.num_runs, a.num_q_heads, a.num_kv_heads, a.head_dim, a.page_size = 1, 1, 8, 2, 128, 16
        a.softmax_scale, a.rope_theta, a.splits = 0.1, 10000.0, 1
        for name, value in changes.items():
            setattr(a, name, value)
        code = lib.fk_page_decode_forward(ctypes.byref(a))
        return code, lib.fk_page_decode_last_error().decode()

    for changes, message in [
        (dict(batch=0), "empty inputs"), (dict(num_runs=-1), "num_runs must be non-negative"),
        (dict(head_dim=96), "head_dim 64 or 128"), (dict(page_size=8), "page_size 16 or 32"),
        (dict(num_q_heads=7), "divisible by num_kv_heads"), (dict(group_tile=3), "group_tile must be one of"),
        (dict(kv_format=5), "unsupported kv_format"), (dict(kv_format=2), "need key_scales and value_scales"),
        (dict(splits=65), "splits must be in"), (dict(query=4100), "16-byte aligned"), (dict(output=0), "must not be NULL"),
        (dict(rope_theta=0.0), "rope_theta positive"), (dict(flags=6), "unknown bits in flags"),
    ]:
        code, text = call(**changes)
        assert code == pdc.ERR_INVALID_ARGUMENT and message in text, (changes, text)
    with pytest.raises(ValueError):
        pdc.check(pdc.ERR_INVALID_ARGUMENT)
    assert lib.fk_page_decode_workspace_bytes(0, 8, 2, 128) == 0
    assert lib.fk_page_decode_workspace_bytes(4, 32, 8, 128) >= 64 * 1024
    assert lib.fk_page_decode_set_launch_config(13, 0) == pdc.ERR_INVALID_ARGUMENT
    assert lib.fk_page_decode_set_launch_config(0, 0) == pdc.OK


def test_native_module_exposes_the_reference_name_and_keywords() -> None:
    from fast_kernels.native import native_module

    doc = native_module().clustered_page_decode_forward.__doc__
    for keyword in ("query_ptr", "key_scales_ptr", "run_last_page_lens_ptr", "request_run_offsets_ptr", "group_tile",
                    "use_clustered_kernel", "cluster_size", "kv_format", "keys_are_rotated", "softmax_scale",
                    "rope_theta", "stream_ptr"):
        assert keyword in doc
    assert KV_IDS == ops.KV_FORMAT_IDS
