#!/usr/bin/env python3
"""Runs one paged-KV decode attention problem a few times through the C ABI -- the small, fixed
workload to put under a profiler
(``ncu -k regex:page_decode ... python run_page_decode.py 16 32 8 128 16 4096 bf16_kv 3``).

    run_page_decode.py BATCH Q_HEADS KV_HEADS HEAD_DIM PAGE_SIZE MAX_LEN bf16_kv|fp8_kv|int8_kv LAUNCHES [WARPS STAGES [SPLITS]]
                       [--shared-prefix TOKENS] [--rotated-keys]

Sequence lengths are drawn within one page of MAX_LEN, the page table is fragmented by a seeded
permutation. The optional numbers override the launch plan (fk_page_decode_set_launch_config and
the `splits` argument). With --shared-prefix every request repeats the first request's first TOKENS
tokens and identical pages are stored once (a prompt prefix shared through the page table). With
--rotated-keys the pages hold keys with their rotary embedding applied (bf16 pages then take the
tensor-core form of the kernel). Prints the launch plan, the time per launch (CUDA events around the whole
burst, so launch overhead is in it) and the device status word.
"""

from __future__ import annotations

import ctypes
import importlib
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "src"))

import torch  # noqa: E402
from fast_kernels import page_decode_capi as pdc  # noqa: E402


def main() -> int:
    rotated = "--rotated-keys" in sys.argv
    if rotated:
        sys.argv.remove("--rotated-keys")
    shared_tokens = 0
    if "--shared-prefix" in sys.argv:
        at = sys.argv.index("--shared-prefix")
        shared_tokens = int(sys.argv[at + 1])
        del sys.argv[at : at + 2]
    if len(sys.argv) < 9:
        print(__doc__)
        return 2
    batch, q_heads, kv_heads, dim, page, max_len = (int(x) for x in sys.argv[1:7])
    layout, launches = sys.argv[7], int(sys.argv[8])
    ops = importlib.import_module("fast_kernels.ops.clustered_page_decode")
    lib = pdc.load_library()
    if len(sys.argv) >= 11:
        pdc.check(lib.fk_page_decode_set_launch_config(int(sys.argv[9]), int(sys.argv[10])))
    splits = int(sys.argv[11]) if len(sys.argv) >= 12 else 0
    generator = torch.Generator().manual_seed(1)
    lens = torch.randint(max(page, max_len - page + 1), max_len + 1, (batch,), generator=generator, dtype=torch.int32)
    query = torch.randn((batch, q_heads, dim), generator=generator).to(torch.bfloat16).cuda()
    torch.manual_seed(2)
    keys = torch.randn((batch, kv_heads, max_len, dim), device="cuda").to(torch.bfloat16)
    values = torch.randn((batch, kv_heads, max_len, dim), device="cuda").to(torch.bfloat16)
    build = {"bf16_kv": ops.pack_paged_kv_bf16, "fp8_kv": ops.quantize_paged_kv_fp8,
             "int8_kv": ops.quantize_paged_kv_int8}[layout]
    if shared_tokens > 0:
        keys[1:, :, :shared_tokens] = keys[0, :, :shared_tokens]
        values[1:, :, :shared_tokens] = values[0, :, :shared_tokens]
    cache = build(keys, values, lens, page_size=page, fragment_pages=True, seed=1,
                  deduplicate_identical_pages=shared_tokens > 0, key_rope_theta=10000.0 if rotated else None)
    del keys, values
    plan = ops.plan_clustered_page_decode(page_table=cache.page_table, seq_lens=cache.seq_lens, num_q_heads=q_heads,
                                          num_kv_heads=kv_heads, head_dim=dim, page_size=page, kv_layout=layout,
                                          use_cache=False)
    descriptors = plan.device_tensors(query.device)
    workspace = torch.zeros(int(lib.fk_page_decode_workspace_bytes(batch, q_heads, kv_heads, dim)), dtype=torch.uint8,
                            device="cuda")
    out = torch.empty_like(query)
    a = pdc.PageDecodeArgs()
    a.query, a.output = query.data_ptr(), out.data_ptr()
    a.key_pages, a.value_pages = cache.key_pages.data_ptr(), cache.value_pages.data_ptr()
    a.key_scales = 0 if cache.key_scales is None else cache.key_scales.data_ptr()
    a.value_scales = 0 if cache.value_scales is None else cache.value_scales.data_ptr()
    for name in ("run_base_pages", "run_page_counts", "run_logical_starts", "run_last_page_lens",
                 "request_run_offsets", "seq_lens"):
        setattr(a, name, descriptors[name].data_ptr())
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.batch, a.num_runs, a.num_q_heads, a.num_kv_heads, a.head_dim, a.page_size = batch, plan.num_runs, q_heads, kv_heads, dim, page
    a.kv_format, a.splits, a.max_pages_hint = ops.KV_FORMAT_IDS[layout], splits, plan.max_pages
    a.keys_are_rotated = int(rotated)
    a.softmax_scale, a.rope_theta = dim**-0.5, 10000.0
    a.stream = int(torch.cuda.current_stream().cuda_stream)
    pdc.check(lib.fk_page_decode_forward(ctypes.byref(a)))
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(launches):
        pdc.check(lib.fk_page_decode_forward(ctypes.byref(a)))
    stop.record()
    torch.cuda.synchronize()
    tokens = int(lens.sum())
    print("plan", pdc.describe_plan(a), "physical pages", cache.total_pages)
    print(f"context tokens {tokens}, {start.elapsed_time(stop) * 1e3 / max(1, launches):.1f} us per launch, "
          f"device status {pdc.device_status()}, max |y| {float(out.float().abs().max()):.4f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
