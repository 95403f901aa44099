"""Shared-prefix paged decode, the parts that need no GPU: the planner against descriptor tables the
reference's own `plan_prefix_union_decode` produced (tests/golden/prefix_union_*.npz, written by
tests/golden/make_page_decode_golden.py), the plan's bookkeeping, argument errors, and the native
module's contract for the kernel entry point."""

from __future__ import annotations

import importlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
union = importlib.import_module("fast_kernels.ops.prefix_union_decode")
CASES = json.loads((GOLDEN / "prefix_union_manifest.json").read_text())


def _plan(meta, case, **kwargs):
    return union.plan_prefix_union_decode(
        page_table=torch.from_numpy(case["page_table"].copy()), seq_lens=torch.from_numpy(case["seq_lens"].copy()),
        num_q_heads=meta["num_q_heads"], num_kv_heads=meta["num_kv_heads"], head_dim=meta["head_dim"],
        page_size=meta["page_size"], kv_layout=meta["layout"], keys_are_rotated=True, use_cache=False, **kwargs)


@pytest.mark.parametrize("meta", CASES, ids=[m["name"] for m in CASES])
def test_planner_reproduces_the_reference_tables(meta) -> None:
    with np.load(GOLDEN / f"prefix_union_{meta['name']}.npz") as data:
        case = {key: data[key] for key in data.files}
    plan = _plan(meta, case)
    for name in ("tasks", "shared_pages", "tail_pages", "consumers"):
        got = getattr(plan, f"{name}_cpu").numpy()
        assert got.dtype == np.int32 and np.array_equal(got, case[name]), name
    assert np.array_equal(plan.fallback_plan.run_base_pages_cpu.numpy(), case["fallback_run_base_pages"])
    assert plan.num_tasks == meta["num_tasks"] and plan.cluster_size == meta["cluster_size"]
    assert plan.estimated_saved_hbm_bytes == meta["estimated_saved_hbm_bytes"]
    # no device of compute capability 12 here (nor on a B200): the reference plans the fallback
    assert plan.launch_mode == meta["launch_mode"] == "fallback"


def test_tables_describe_the_sharing() -> None:
    """Two requests that start with the same two pages and one that does not, one kv head, two
    query heads: one task for the pair (2 shared pages, 4 consumers), one for the loner."""
    table = torch.tensor([[7, 3, 9, -1], [7, 3, 4, 5], [1, 2, 6, -1]], dtype=torch.int32)
    lens = torch.tensor([40, 64, 33], dtype=torch.int32)
    plan = union.plan_prefix_union_decode(page_table=table, seq_lens=lens, num_q_heads=2, num_kv_heads=1, head_dim=64,
                                          page_size=16, kv_layout="bf16_kv", keys_are_rotated=True, use_cache=False)
    assert plan.tasks_cpu.tolist() == [[0, 2, 0, 4, 0, 0, 0, 0], [2, 0, 4, 2, 0, 0, 0, 0]]
    assert plan.shared_pages_cpu.tolist() == [[7, 16], [3, 16]]
    # consumers: request 0 heads 0, 1 (tail = page 9 with 8 tokens at logical page 2), request 1 ..., then request 2
    assert plan.consumers_cpu.tolist()[0] == [0, 0, 0, 39, 1, 0, 0, 0]
    assert plan.consumers_cpu.tolist()[2] == [2, 2, 2, 63, 2, 0, 0, 0]
    assert plan.tail_pages_cpu.tolist()[0] == [9, 8 | (2 << 16)]
    assert plan.tail_pages_cpu.tolist()[2:4] == [[4, 16 | (2 << 16)], [5, 16 | (3 << 16)]]
    assert plan.consumers_cpu.tolist()[4] == [4, 4, 6, 32, 3, 0, 0, 0]
    assert plan.estimated_saved_hbm_bytes == 3 * 2 * (2 * 16 * 64 * 2)
    metrics_cache = type("C", (), {"kv_layout": "bf16_kv", "seq_lens": lens, "num_kv_heads": 1, "head_dim": 64})()
    metrics = union.estimate_prefix_union_decode_metrics(metrics_cache, plan)
    assert metrics["estimated_saved_hbm_bytes"] == float(plan.estimated_saved_hbm_bytes)
    assert metrics["workspace_bytes_per_token"] == 0.0


def test_argument_errors() -> None:
    table, lens = torch.zeros((1, 2), dtype=torch.int32), torch.tensor([20], dtype=torch.int32)
    common = dict(page_table=table, seq_lens=lens, num_q_heads=4, num_kv_heads=2, head_dim=64, page_size=16,
                  kv_layout="bf16_kv", keys_are_rotated=True, use_cache=False)
    with pytest.raises(ValueError, match="min_consumers must be >= 2"):
        union.plan_prefix_union_decode(**{**common, "min_consumers": 1})
    with pytest.raises(ValueError, match="min_shared_pages must be >= 1"):
        union.plan_prefix_union_decode(**{**common, "min_shared_pages": 0})
    with pytest.raises(ValueError, match="cluster_size must be one of"):
        union.plan_prefix_union_decode(**{**common, "cluster_size": 3})
    with pytest.raises(ValueError, match="head_dim must be 64 or 128"):
        union.plan_prefix_union_decode(**{**common, "head_dim": 80})


def test_native_entry_point_keeps_the_reference_contract_below_compute_capability_12() -> None:
    """Exported under the reference's name with its keywords; zero tasks is a no-op; anything else is
    the std::invalid_argument the reference's launcher throws on such a device."""
    from fast_kernels.native import native_module

    native = native_module()
    for keyword in ("tasks_ptr", "shared_pages_ptr", "tail_pages_ptr", "consumers_ptr", "scheduler_counter_ptr",
                    "num_tasks", "num_pages", "cluster_size", "keys_are_rotated"):
        assert keyword in native.prefix_union_decode_forward.__doc__
    zeros = [0] * 11
    native.prefix_union_decode_forward(*zeros, 0, 1, 8, 2, 128, 16, 1, 0, 1, 0.1, 10000.0, 0)
    with pytest.raises(ValueError, match="compute capability 12"):
        native.prefix_union_decode_forward(*zeros, 3, 1, 8, 2, 128, 16, 1, 0, 1, 0.1, 10000.0, 0)
