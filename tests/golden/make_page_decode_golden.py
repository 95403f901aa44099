"""Generates tests/golden/page_decode_*.npz by running the REFERENCE's own Python for the paged-KV
decode attention (SamMausberg/fast-kernels) on CPU tensors.

The reference stores no golden vectors for this op: its GPU tests
(tests/gpu/test_clustered_page_decode.py:113-156 there) build a cache with `pack_paged_kv_bf16` /
`quantize_paged_kv_int8` / `quantize_paged_kv_fp8`, plan with `plan_clustered_page_decode` and
compare the kernel with `reference_clustered_page_decode`. This script imports exactly those
functions from a reference checkout, calls them on CPU (none of them needs a GPU) with the tests'
value recipe (`_make_case_inputs`, :42-66: randn query / keys / values in bf16, sequence lengths
within one page of the maximum), and stores inputs, the cache bytes, the plan arrays and the
expected output as bit patterns. It needs the checkout; the tests that consume the fixtures do
not.

    python tests/golden/make_page_decode_golden.py --reference <path of the reference checkout>

Also writes tests/golden/prefix_union_*.npz: page tables with shared prefixes and the four
descriptor tables the reference's `plan_prefix_union_decode` makes of them.

Cases: the shapes of the reference's GPU tests scaled to CPU-friendly sizes, each layout, keys
rotated ahead of time or not, both page sizes and head dims, fragmented and contiguous page
tables, de-duplicated pages.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = [
    # name, layout, batch, q_heads, kv_heads, head_dim, max_seq_len, page_size, key_rope_theta, fragment, dedup
    ("bf16_d64_p16_g1", "bf16_kv", 2, 2, 2, 64, 64, 16, None, True, False),
    ("bf16_d64_p16_g4", "bf16_kv", 2, 8, 2, 64, 128, 16, None, True, False),
    ("int8_d128_p32_g8", "int8_kv", 2, 8, 1, 128, 160, 32, None, True, False),
    ("bf16_d128_p32_g32", "bf16_kv", 2, 32, 1, 128, 160, 32, None, True, False),
    ("fp8_d128_p32_g8", "fp8_kv", 2, 8, 1, 128, 160, 32, None, True, False),
    ("bf16_d64_p16_g4_rot", "bf16_kv", 2, 8, 2, 64, 128, 16, 10000.0, True, False),
    ("fp8_d64_p16_g4_rot", "fp8_kv", 2, 8, 2, 64, 128, 16, 10000.0, True, False),
    ("int8_d128_p32_g32_rot", "int8_kv", 2, 32, 1, 128, 160, 32, 10000.0, True, False),
    ("bf16_d128_p16_g2_contig", "bf16_kv", 3, 4, 2, 128, 100, 16, None, False, False),
    ("int8_d64_p32_g2_dedup", "int8_kv", 3, 4, 2, 64, 96, 32, None, True, True),
]


# Shared-prefix cases for the planner of prefix_union_decode (the reference's
# tests/gpu/test_prefix_union_decode.py:48-98 recipe: the requests of a group repeat their leader's
# first pages, pages are de-duplicated and fragmented with seed 3, keys rotated ahead of time):
# name, batch, q_heads, kv_heads, head_dim, max_seq_len, page_size, shared_prefix_pages, prefix_group_size, layout
PREFIX_CASES = [
    ("gqa4_prefix4", 8, 8, 2, 64, 160, 16, 4, 4, "bf16_kv"),
    ("mqa8_prefix3_odd_groups", 7, 8, 1, 64, 200, 32, 3, 3, "int8_kv"),
    ("gqa2_prefix2_pairs", 6, 4, 2, 64, 96, 16, 2, 2, "fp8_kv"),
    ("no_sharing", 3, 4, 2, 64, 80, 16, 0, 1, "bf16_kv"),
]


def _load_reference(reference: Path):
    sys.path.insert(0, str(reference / "src"))
    if "matplotlib" not in sys.modules:  # imported by the reference's reporting package, not needed here
        fake = types.ModuleType("matplotlib")
        fake.use = lambda *a, **k: None  # type: ignore[attr-defined]
        pyplot = types.ModuleType("matplotlib.pyplot")
        fake.pyplot = pyplot  # type: ignore[attr-defined]
        sys.modules["matplotlib"] = fake
        sys.modules["matplotlib.pyplot"] = pyplot
    import importlib  # noqa: PLC0415

    # the package re-exports a function of the same name, so fetch the module itself
    return importlib.import_module("fast_kernels.ops.clustered_page_decode")


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def _raw(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return _bits(t)
    return t.contiguous().view(torch.uint8).numpy().copy()


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--reference", default=os.environ.get("FK_REFERENCE_ROOT"),
                        help="path of the reference checkout (or set FK_REFERENCE_ROOT)")
    ns = parser.parse_args()
    if not ns.reference:
        parser.error("--reference (or FK_REFERENCE_ROOT) is required")
    ops = _load_reference(Path(ns.reference))
    manifest = []
    for name, layout, batch, q_heads, kv_heads, head_dim, max_seq, page, theta, fragment, dedup in CASES:
        torch.manual_seed(batch + q_heads + kv_heads + head_dim + max_seq + page)  # the tests' seed formula
        query = torch.randn((batch, q_heads, head_dim)).to(torch.bfloat16)
        keys = torch.randn((batch, kv_heads, max_seq, head_dim)).to(torch.bfloat16)
        values = torch.randn((batch, kv_heads, max_seq, head_dim)).to(torch.bfloat16)
        seq_lens = torch.randint(low=max(page, max_seq - page + 1), high=max_seq + 1, size=(batch,), dtype=torch.int32)
        if dedup:  # make some pages identical: the second request repeats the first one's prefix
            keys[1, :, : 2 * page] = keys[0, :, : 2 * page]
            values[1, :, : 2 * page] = values[0, :, : 2 * page]
        build = {"bf16_kv": ops.pack_paged_kv_bf16, "int8_kv": ops.quantize_paged_kv_int8,
                 "fp8_kv": ops.quantize_paged_kv_fp8}[layout]
        cache = build(keys, values, seq_lens, page_size=page, fragment_pages=fragment, seed=1,
                      key_rope_theta=theta, deduplicate_identical_pages=dedup)
        plan = ops.plan_clustered_page_decode(
            page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=q_heads, num_kv_heads=kv_heads,
            head_dim=head_dim, page_size=page, kv_layout=layout, use_cache=False)
        expected = ops.reference_clustered_page_decode(query, cache)
        arrays = {
            "query": _bits(query), "keys": _bits(keys), "values": _bits(values),
            "seq_lens": seq_lens.numpy().copy(),
            "key_pages": _raw(cache.key_pages), "value_pages": _raw(cache.value_pages),
            "page_table": cache.page_table.numpy().copy(),
            "run_base_pages": plan.run_base_pages_cpu.numpy().copy(),
            "run_page_counts": plan.run_page_counts_cpu.numpy().copy(),
            "run_logical_starts": plan.run_logical_starts_cpu.numpy().copy(),
            "run_last_page_lens": plan.run_last_page_lens_cpu.numpy().copy(),
            "request_run_offsets": plan.request_run_offsets_cpu.numpy().copy(),
            "expected": _bits(expected),
        }
        if cache.key_scales is not None:  # for bf16 pages the unquantised pages ARE key_pages / value_pages
            arrays["reference_key_pages"] = _bits(cache.reference_key_pages)
            arrays["reference_value_pages"] = _bits(cache.reference_value_pages)
            arrays["key_scales"] = cache.key_scales.numpy().copy()
            arrays["value_scales"] = cache.value_scales.numpy().copy()
        np.savez_compressed(HERE / f"page_decode_{name}.npz", **arrays)
        manifest.append({
            "name": name, "layout": layout, "batch": batch, "num_q_heads": q_heads, "num_kv_heads": kv_heads,
            "head_dim": head_dim, "max_seq_len": max_seq, "page_size": page, "key_rope_theta": theta,
            "fragment_pages": fragment, "deduplicate_identical_pages": dedup, "seed": 1,
            "plan": {"max_pages": plan.max_pages, "group_tile": plan.group_tile, "q_head_tiles": plan.q_head_tiles,
                     "cluster_size": plan.cluster_size, "launch_mode": plan.launch_mode},
            "total_pages": cache.total_pages,
        })
        print(name, "pages", cache.total_pages, "runs", plan.num_runs)
    (HERE / "page_decode_manifest.json").write_text(json.dumps(manifest, indent=1) + "\n")

    import importlib  # noqa: PLC0415

    union = importlib.import_module("fast_kernels.ops.prefix_union_decode")
    prefix_manifest = []
    for name, batch, q_heads, kv_heads, head_dim, max_seq, page, shared_pages, group, layout in PREFIX_CASES:
        torch.manual_seed(batch + q_heads + kv_heads + head_dim + max_seq + page + shared_pages + group)
        shared_tokens = shared_pages * page
        keys = torch.randn((batch, kv_heads, max_seq, head_dim)).to(torch.bfloat16)
        values = torch.randn((batch, kv_heads, max_seq, head_dim)).to(torch.bfloat16)
        seq_lens = torch.randint(low=max(page, shared_tokens + 1), high=max_seq + 1, size=(batch,), dtype=torch.int32)
        for start in range(0, batch, group):
            for follower in range(start + 1, min(batch, start + group)):
                keys[follower, :, :shared_tokens] = keys[start, :, :shared_tokens]
                values[follower, :, :shared_tokens] = values[start, :, :shared_tokens]
        build = {"bf16_kv": ops.pack_paged_kv_bf16, "int8_kv": ops.quantize_paged_kv_int8,
                 "fp8_kv": ops.quantize_paged_kv_fp8}[layout]
        cache = build(keys, values, seq_lens, page_size=page, fragment_pages=True, seed=3, key_rope_theta=10000.0,
                      deduplicate_identical_pages=True)
        plan = union.plan_prefix_union_decode(
            page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=q_heads, num_kv_heads=kv_heads,
            head_dim=head_dim, page_size=page, kv_layout=layout, keys_are_rotated=True, use_cache=False)
        np.savez_compressed(
            HERE / f"prefix_union_{name}.npz", page_table=cache.page_table.numpy().copy(),
            seq_lens=seq_lens.numpy().copy(), tasks=plan.tasks_cpu.numpy().copy(),
            shared_pages=plan.shared_pages_cpu.numpy().copy(), tail_pages=plan.tail_pages_cpu.numpy().copy(),
            consumers=plan.consumers_cpu.numpy().copy(),
            fallback_run_base_pages=plan.fallback_plan.run_base_pages_cpu.numpy().copy())
        prefix_manifest.append({
            "name": name, "batch": batch, "num_q_heads": q_heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
            "max_seq_len": max_seq, "page_size": page, "shared_prefix_pages": shared_pages,
            "prefix_group_size": group, "layout": layout, "total_pages": cache.total_pages,
            "launch_mode": plan.launch_mode, "cluster_size": plan.cluster_size,
            "estimated_saved_hbm_bytes": plan.estimated_saved_hbm_bytes, "num_tasks": plan.num_tasks,
            "metrics": union.estimate_prefix_union_decode_metrics(cache, plan),
        })
        print(name, "tasks", plan.num_tasks, "saved", plan.estimated_saved_hbm_bytes, "pages", cache.total_pages)
    (HERE / "prefix_union_manifest.json").write_text(json.dumps(prefix_manifest, indent=1) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
